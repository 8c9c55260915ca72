// Prefill / batched-decode GEMM on the 5th-generation tensor cores:
//   C[t][n] = sum_k X[t][k] * W[k][n],  X fp16 activations, W INT4 (group-wise scale/zero),
//   fp32 accumulation in tensor memory.
//
// Replaces the reference's prefill GEMM family (reference:
// src/kernels/gemm_int4_prefill_hip.hip:27, gemm_int4_prefill_v2.hip:41,
// gemm_fp16_prefill.hip:47, gemm_fp16_prefill_silu_dual.hip:62, src/asm/gemm_*.s), which
// runs 64x64x16 tiles on vector ALUs.
//
// One CTA computes a [128 outputs x T tokens] tile (T <= 512, all of tensor memory):
//   * the WEIGHT tile is the MMA's A operand (M = 128 outputs), the activations are the B
//     operand (N = tokens, any multiple of 16 up to 256 per instruction), so a weight tile is
//     dequantised once and used for every token, and a batch of 16..80 rows costs no padding;
//   * warps 0-15 (two groups of 8, alternating k-blocks) stream the packed nibbles through a
//     cp.async ring (same fragment order the decode GEMV uses), expand them to fp16 with the
//     0x6400 trick, apply (q - zero) * scale and store the tile into shared memory in the
//     K-major 128-byte-swizzled layout tcgen05 reads;
//   * warp 16 brings the activation tile with TMA (cp.async.bulk.tensor, 128-byte swizzle, no
//     cluster broadcast) onto the stage's mbarrier; with dense fp16 weights (the lm_head of many
//     rows) it loads the weight tile the same way and the dequantising warps idle;
//   * warp 17 issues tcgen05.mma (cta_group::1, kind::f16) on shared-memory descriptors and
//     releases stages with tcgen05.commit; both single-lane roles keep their warp converged and
//     elect a lane only around the tcgen05 / TMA instructions;
//   * warps 0-15 then read the accumulators back with tcgen05.ld and run the epilogue: store,
//     SiLU(gate)*up for the interleaved gate/up matrix, residual add, or -- under tensor
//     parallelism -- stores straight into the staging buffer of the rank that reduces that
//     slice of the output (reduce-scatter fused into the GEMM).
// Every mbarrier wait is bounded; on expiry the kernel records a status, skips the rest of
// its work, releases its tensor memory and returns.
#include <cuda.h>
#include "kernels.cuh"
#include "gemm_tc.cuh"
#include "tc_util.cuh"

#define TC_PRODUCERS 16           // dequantising warps (also the epilogue warps): two groups of 8, group g takes
                                  // the k-blocks of parity g, so two k-blocks are being dequantised at any time
#define TC_GROUP_WARPS 8
#define TC_THREADS ((TC_PRODUCERS + 2) * 32)
#define TC_BK 64                 // k per stage (128 bytes of fp16: one swizzle row)
#define TC_BM 128                // outputs per CTA (MMA M)
#define TC_A_BYTES (TC_BM * TC_BK * 2)
#define TC_RING_OF(pair) ((pair) ? 2 : 3)     // own k-blocks of packed weights + scales in flight per producer thread (cp.async);
                                              // CTA pairs trade one for two more pipeline stages (their token stages are half as large)

// ---------------------------------------------------------------------------
// Kernel
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t tc_nib_lo(uint32_t w) {
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(r) : "r"(w));
    return r;
}
__device__ __forceinline__ uint32_t tc_nib_hi(uint32_t w) {
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(r) : "r"(w));
    return r;
}

// PAIR: the kernel of CTA pairs is an instantiation of its own: a kernel that contains cta_group::2 instructions
// cannot be launched without a cluster (the plain launch is refused with "invalid cluster size").
template <bool PAIR>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_int4_tc_kernel(const GemmTcParams p, const __grid_constant__ CUtensorMap xmap,
                    const __grid_constant__ CUtensorMap wmap) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the dynamic window is only guaranteed 16-byte aligned: align to the 1024-byte swizzle atom by hand
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.stages;
    const int t0 = blockIdx.y * p.t_tile;
    const int Tp = (min(p.t_tile, p.T - t0) + 15) & ~15;          // token columns of this CTA
    const int boxes = (Tp + 63) / 64;
    // (CTA pairs: a CTA stages only its half of the token rows)
    const int b_stage_bytes = ((p.t_tile + 63) / 64) * 64 * 128 / (PAIR ? 2 : 1);
    // MH = 2: the CTA owns 256 outputs as two M = 128 accumulators that share every activation tile (half the
    // activation bytes per FLOP, one pass of the dequantising warps per 256 outputs); all 16 producer warps
    // then work on the same k-block
    // pair: two CTAs of a cluster (adjacent output tiles) run their MMAs as one cta_group::2 instruction stream,
    // M = 256 over the two SMs: each CTA dequantises its own 128 weight rows and loads only ITS half of every
    // 256-token operand tile, so the shared-memory traffic of the token operand per SM halves
    constexpr bool pair = PAIR;
    constexpr int TC_RING = TC_RING_OF(PAIR);
    uint32_t crank = 0u;
    if constexpr (PAIR) crank = cluster_ctarank();
    const int MH = p.m_halves == 2 ? 2 : 1;
    const int a_bytes = MH * TC_A_BYTES;
    unsigned char* sA = smem;
    unsigned char* sB = smem + (size_t)S * a_bytes;
    uint64_t* bars = (uint64_t*)(sB + (size_t)S * b_stage_bytes);
    uint64_t* full = bars;              // [S] operands of the stage are in place: one arrival per producer warp of
                                        // the stage's group (INT4 weights) + 1 arrival with the TMA transaction bytes
    uint64_t* empty = bars + S;         // [S] 1 arrival (tcgen05.commit)
    uint64_t* acc_full = bars + 2 * S;  // 1 arrival
    uint64_t* peer_full = bars + 2 * S + 1;   // [S] pair mode, leader CTA: the peer's operands of the stage are in place
    uint32_t* tmem_slot = (uint32_t*)(bars + 3 * S + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    uint4* wring = (uint4*)(((uintptr_t)(tmem_slot + 2) + 15) & ~(uintptr_t)15);   // [TC_RING][2][512 producer threads]: 16 B of nibbles, 2 x 8 B scale/zero

    int tmem_cols = 32;
    while (tmem_cols < Tp) tmem_cols <<= 1;
    if (MH == 2) tmem_cols = 512;                  // accumulator h at column 256 h (Tp <= 256)

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], p.dense ? 1 : (MH == 2 ? TC_PRODUCERS : TC_GROUP_WARPS) + 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        for (int s = 0; s < S; ++s) mbar_init(&peer_full[s], 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if constexpr (PAIR) cluster_sync_all();       // both CTAs' barriers exist before anyone signals the other
    if (warp == TC_PRODUCERS) {
        if constexpr (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         :: "r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         :: "r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // split-K: this CTA's k-blocks are [kb_lo, kb_lo + KB) of the p.KB blocks of the matrix
    const int per_kb = (p.KB + (int)gridDim.z - 1) / (int)gridDim.z;
    const int kb_lo = (int)blockIdx.z * per_kb;
    const int KB = max(0, min(p.KB, kb_lo + per_kb) - kb_lo);

    // Every role walks the stages with running counters (stage index, phase bit, addresses).  The
    // loops of the single-thread roles are chains of dependent instructions, so each instruction
    // taken out of them shortens the time per k-block directly.
    if (warp < TC_PRODUCERS) {
        // ================= weight producers =================
        // warp w owns the 16-row tile w of the CTA's 128 outputs: one 16-byte load per k-block and lane
        const int g = lane >> 2, t = lane & 3;
        // MH = 1: two groups of 8 warps take alternate k-blocks; MH = 2: one group of 16 takes every k-block
        const int grp = MH == 2 ? 0 : warp >> 3, w8 = MH == 2 ? warp : warp & 7;
        const int kstep = MH == 2 ? 1 : 2;
        const int wt = blockIdx.x * (2 * MH) + (w8 >> 2);
        const int ti = w8 & 3;
        const bool dense = p.dense != 0;          // fp16 weights arrive by TMA: nothing to dequantise
        const __half2 sixteenth = __float2half2_rn(0.0625f);
        const __half2 k1024 = __float2half2_rn(1024.f), k64 = __float2half2_rn(64.f);
        // swizzled byte offsets of this lane's stores: row & 7 == g for both of its rows
        const uint32_t row_lo_off = (uint32_t)(w8 * 16 + g) * 128 + t * 4;
        uint32_t sw[8];
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) sw[c8] = (uint32_t)((c8 ^ g) << 4);
        // packed weights and their scale/zero pairs stream through a cp.async ring: TC_RING-1 of
        // the group's k-blocks are always in flight, each thread later reads back only what it copied
        uint4* my_ring = wring + tid;
        const uint4* gq = dense ? nullptr : p.qfrag + ((size_t)wt * p.KB * 4 + ti) * 32 + lane + (size_t)(kb_lo + grp) * 128;
        const uint2* gs = dense ? nullptr : p.szfrag + ((size_t)wt * p.G * 4 + ti) * 8 + g;
        const uint32_t gq_step = 128u * kstep;
        const int c_step = 2 * kstep;
        int c_issue = p.off32 + 2 * (kb_lo + grp);          // 32-k chunk counter of the next k-block to issue
        int slot_issue = 0;
        auto issue = [&]() {
            uint4* dst = my_ring + slot_issue * 1024;
            cp_async16(dst, gq);
            cp_async8((uint2*)(dst + 512), gs + (size_t)(c_issue >> p.gshift) * 32);
            cp_async8((uint2*)(dst + 512) + 1, gs + (size_t)((c_issue + 1) >> p.gshift) * 32);
            gq += gq_step; c_issue += c_step;
            slot_issue = slot_issue == TC_RING - 1 ? 0 : slot_issue + 1;
        };
#pragma unroll
        for (int i = 0; i < TC_RING - 1; ++i) {
            if (grp + kstep * i < KB && !dense) issue();
            cp_async_commit();
        }
        bool ok = true;
        int st = grp, slot = 0;
        uint32_t ph = 0;
        unsigned char* a_stage = sA + (size_t)grp * a_bytes + row_lo_off;
        for (int kb = grp; kb < KB && !dense; kb += kstep) {
            if (kb + kstep * (TC_RING - 1) < KB) issue();
            cp_async_commit();
            cp_async_wait<TC_RING - 1>();
            const uint4 wv = my_ring[slot * 1024];
            const uint4 szq = my_ring[slot * 1024 + 512];
            slot = slot == TC_RING - 1 ? 0 : slot + 1;
            {   // one lane polls: many pollers on one barrier slow the arrivals down
                int o = 1;
                if (lane == 0) o = mbar_wait(&empty[st], ph ^ 1, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, o, 0) != 0;
            }
            if (!ok) break;
            unsigned char* a_lo = a_stage;
            unsigned char* a_hi = a_stage + 8 * 128;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint2 sz = j ? make_uint2(szq.z, szq.w) : make_uint2(szq.x, szq.y);
                const __half2 s2 = *(const __half2*)&sz.x, z2 = *(const __half2*)&sz.y;
                const __half2 s_lo = __half2half2(__low2half(s2)), s_hi = __half2half2(__high2half(s2));
                const __half2 z_lo = __half2half2(__low2half(z2)), z_hi = __half2half2(__high2half(z2));
                const __half2 cl_lo = __hadd2(k1024, z_lo), cl_hi = __hadd2(k1024, z_hi);                  // 1024 + zero
                const __half2 ch_lo = __hneg2(__hadd2(k64, z_lo)), ch_hi = __hneg2(__hadd2(k64, z_hi));   // -(64 + zero)
                const uint32_t w0 = j ? wv.z : wv.x, w1 = j ? wv.w : wv.y;
                auto deq_lo = [&](uint32_t x, __half2 c, __half2 sc) {
                    uint32_t r = tc_nib_lo(x);
                    return __hmul2(__hsub2(*(__half2*)&r, c), sc);
                };
                auto deq_hi = [&](uint32_t x, __half2 c, __half2 sc) {
                    uint32_t r = tc_nib_hi(x);
                    return __hmul2(__hfma2(*(__half2*)&r, sixteenth, c), sc);
                };
                // k = 32 j + 8 m + 2 t: the 16-byte column group is 4 j + m
                *(__half2*)(a_lo + sw[4 * j + 0]) = deq_lo(w0, cl_lo, s_lo);
                *(__half2*)(a_hi + sw[4 * j + 0]) = deq_lo(w0 >> 8, cl_hi, s_hi);
                *(__half2*)(a_lo + sw[4 * j + 2]) = deq_hi(w0, ch_lo, s_lo);
                *(__half2*)(a_hi + sw[4 * j + 2]) = deq_hi(w0 >> 8, ch_hi, s_hi);
                *(__half2*)(a_lo + sw[4 * j + 1]) = deq_lo(w1, cl_lo, s_lo);
                *(__half2*)(a_hi + sw[4 * j + 1]) = deq_lo(w1 >> 8, cl_hi, s_hi);
                *(__half2*)(a_lo + sw[4 * j + 3]) = deq_hi(w1, ch_lo, s_lo);
                *(__half2*)(a_hi + sw[4 * j + 3]) = deq_hi(w1 >> 8, ch_hi, s_hi);
            }
            fence_proxy_async_smem();           // generic-proxy stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[st]);
            st += kstep; a_stage += kstep * a_bytes;  // two groups: S is even, a group keeps to the stages of its parity
            if (st >= S) { st -= S; ph ^= 1; a_stage = sA + (size_t)st * a_bytes + row_lo_off; }
        }
        cp_async_wait<0>();
        // ================= epilogue =================
        if (ok) ok = mbar_wait(acc_full, 0, abort_flag);
        tc_fence_after();
        if (ok) {
            const int lg = warp & 3;               // tensor-memory lane group this warp may read
            for (int hc = 0; hc < MH; ++hc)
            for (int c0 = (warp >> 2) * 32; c0 < Tp; c0 += (TC_PRODUCERS / 4) * 32) {
                const int n = blockIdx.x * (TC_BM * MH) + hc * TC_BM + lg * 32 + lane;
                uint32_t r[32];
                tc_ld32(tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(hc * 256 + c0), r);
                tc_wait_ld();
                if (p.epi == TC_EPI_SILU_PAIR) {
                    const bool is_gate = (lane & 8) == 0;
                    const int o = blockIdx.x * (TC_BM / 2 * MH) + hc * (TC_BM / 2) + lg * 16 + (lane >> 4) * 8 + (lane & 7);
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        float v = __uint_as_float(r[c]);
                        float up = __shfl_down_sync(0xffffffffu, v, 8);
                        int tt = t0 + c0 + c;
                        if (is_gate && c0 + c < Tp && tt < p.T && o < p.n_valid)
                            ((__half*)p.out)[(size_t)tt * p.ldo + o] = __float2half(silu_f(v) * up);
                    }
                } else if (p.epi == TC_EPI_PUSH_F32) {
                    // plain stores into the owner's memory over NVLink (posted writes, 128 bytes per warp)
                    const size_t poff = (size_t)((*p.epoch + 1u) & 1u) * (size_t)p.part_stride;
#pragma unroll 4
                    for (int c = 0; c < 32; ++c) {
                        int tt = t0 + c0 + c;
                        if (c0 + c < Tp && tt < p.T && n < p.n_valid) {
                            const unsigned e = (unsigned)tt * (unsigned)p.ldo + (unsigned)n;
                            const unsigned i4 = e >> 2, owner = i4 / p.push_per;
                            float* dst = p.push[owner] + poff + ((size_t)p.push_rank * p.push_per + (i4 - owner * p.push_per)) * 4 + (e & 3u);
                            *dst = __uint_as_float(r[c]);
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        int tt = t0 + c0 + c;
                        if (c0 + c < Tp && tt < p.T && n < p.n_valid) {
                            float v = __uint_as_float(r[c]);
                            size_t o = (size_t)tt * p.ldo + n;
                            if (p.epi == TC_EPI_STORE_F16) ((__half*)p.out)[o] = __float2half(v);
                            else if (p.epi == TC_EPI_STORE_F32) ((float*)p.out)[o] = v;
                            else if (gridDim.z > 1) atomicAdd((float*)p.out + o, v);     // split-K partial
                            else ((float*)p.out)[o] += v;
                        }
                    }
                }
            }
        }
    } else if (warp == TC_PRODUCERS) {
        // ================= activation producer (TMA) =================
        {
            const bool dense = p.dense != 0;
            // pair mode: of every 256-token operand tile this CTA loads rows [128 crank, 128 crank + 128)
            const uint32_t tx = (pair ? (uint32_t)(Tp / 2) * 128u : (uint32_t)boxes * 64 * 128) + (dense ? (uint32_t)a_bytes : 0u);
            const int row_w = blockIdx.x * (TC_BM * MH);
            int st = 0;
            uint32_t ph = 0;
            unsigned char* a = sA;
            unsigned char* b = sB;
            for (int kb = 0, kx = kb_lo * TC_BK; kb < KB; ++kb, kx += TC_BK) {
                if (!mbar_wait(&empty[st], ph ^ 1, abort_flag)) break;
                if (elect_one()) {
                    mbar_arrive_expect_tx(&full[st], tx);
                    if (dense) for (int hc = 0; hc < MH; ++hc) tma_load_2d(a + hc * TC_A_BYTES, &wmap, kx, row_w + hc * TC_BM, &full[st]);
                    if (pair) {
                        for (int j = 0; j < Tp / 256; ++j)
                            for (int bx = 0; bx < 2; ++bx)
                                tma_load_2d(b + j * (128 * 128) + bx * (64 * 128), &xmap, kx, t0 + j * 256 + (int)crank * 128 + bx * 64, &full[st]);
                    } else {
                        for (int bx = 0; bx < boxes; ++bx)
                            tma_load_2d(b + bx * (64 * 128), &xmap, kx, t0 + bx * 64, &full[st]);
                    }
                }
                __syncwarp();
                a += a_bytes; b += b_stage_bytes;
                if (++st == S) { st = 0; ph ^= 1; a = sA; b = sB; }
            }
        }
    } else {
        // ================= MMA issuer =================
        {
            const bool dense = p.dense != 0;
            const int n1 = min(Tp, 256), n2 = Tp - n1;
            const uint32_t idesc1 = make_idesc_f16(n1), idesc2 = make_idesc_f16(n2 > 0 ? n2 : 16);
            // descriptors differ between stages and k16 steps only in the start-address field (16-byte units)
            const uint64_t ad0 = make_desc_sw128(smem_u32(sA)), bd0 = make_desc_sw128(smem_u32(sB));
            const uint64_t a_step = (uint64_t)(a_bytes >> 4), b_step = (uint64_t)(b_stage_bytes >> 4), b_half = (256 * 128) >> 4;
            const uint64_t a_half = TC_A_BYTES >> 4;
            uint64_t ad = ad0, bd = bd0;
            int st = 0;
            uint32_t ph = 0;
            bool ok = true;
            const uint32_t idesc_pair = make_idesc_f16_m256(256);
            const uint64_t b_pair_half = (128 * 128) >> 4;
            for (int kb = 0; kb < KB; ++kb) {
                ok = mbar_wait(&full[st], ph, abort_flag);
                if (!ok) break;
                if constexpr (PAIR) {
                    if (crank != 0) {
                        // peer CTA: its operands of the stage are in place: tell the leader, which issues for both
                        if (elect_one()) mbar_arrive_remote(&peer_full[st], 0);
                        __syncwarp();
                        if (++st == S) { st = 0; ph ^= 1; }
                        continue;
                    }
                    ok = mbar_wait_cluster(&peer_full[st], ph, abort_flag);
                    if (!ok) break;
                }
                tc_fence_after();
                if constexpr (PAIR) {
                    if (elect_one()) {
#pragma unroll
                        for (int k16 = 0; k16 < TC_BK / 16; ++k16)
                            for (int j = 0; j < Tp / 256; ++j)
                                tc_mma_f16_pair(tmem_base + 256 * j, ad + 2 * k16, bd + j * b_pair_half + 2 * k16, idesc_pair, (kb | k16) ? 1u : 0u);
                        tc_commit_pair(&empty[st]);
                    }
                    __syncwarp();
                    ad += a_step; bd += b_step;
                    if (++st == S) { st = 0; ph ^= 1; ad = ad0; bd = bd0; }
                    continue;
                }
                if (elect_one()) {
#pragma unroll
                    for (int k16 = 0; k16 < TC_BK / 16; ++k16) {
                        tc_mma_f16(tmem_base, ad + 2 * k16, bd + 2 * k16, idesc1, (kb | k16) ? 1u : 0u);
                        if (MH == 2) tc_mma_f16(tmem_base + 256, ad + a_half + 2 * k16, bd + 2 * k16, idesc1, (kb | k16) ? 1u : 0u);
                        else if (n2 > 0) tc_mma_f16(tmem_base + 256, ad + 2 * k16, bd + b_half + 2 * k16, idesc2, (kb | k16) ? 1u : 0u);
                    }
                    tc_commit(&empty[st]);      // stage reusable once these MMAs have read it
                }
                __syncwarp();
                ad += a_step; bd += b_step;
                if (++st == S) { st = 0; ph ^= 1; ad = ad0; bd = bd0; }
            }
            if constexpr (PAIR) { if (ok && crank == 0 && elect_one()) tc_commit_pair(acc_full); }
            else { if (ok && elect_one()) tc_commit(acc_full); }
            __syncwarp();
        }
    }
    if (*abort_flag && tid == 0 && p.status) atomicExch(p.status, 1);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if constexpr (PAIR) cluster_sync_all();       // neither CTA frees tensor memory (or leaves) while the pair's MMAs or
                                                  // the other CTA's signals may still touch it
    if (warp == TC_PRODUCERS) {
        if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(tmem_cols) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
B2_API size_t b2_gemm_tc_smem(int t_tile, int stages, int m_halves, int ring) {
    size_t b = (size_t)((t_tile + 63) / 64) * 64 * 128;
    return 1024 + (size_t)stages * ((size_t)(m_halves == 2 ? 2 : 1) * TC_A_BYTES + b) + (3 * stages + 1) * 8 + 16 + 16 +
           (size_t)ring * 2 * (TC_PRODUCERS * 32) * 16;
}

// x: [T][ldx] fp16 activations (ldx multiple of 8, base 16-byte aligned).
static int launch_tc(const GemmTcParams* p, const void* w, int ldw, int n_rows_w, const void* x, int ldx,
                     cudaStream_t stream) {
    if (p->T < 1 || p->t_tile < 16 || p->t_tile > 512 || (p->t_tile & 15) || (ldx & 7) || ((uintptr_t)x & 15))
        return cudaErrorInvalidValue;
    EncodeTiledFn enc = get_encode();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)p->K, (cuuint64_t)p->T};
    cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
    cuuint32_t box[2] = {TC_BK, 64};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)x, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    CUtensorMap wmap = map;
    if (w) {
        if ((ldw & 7) || ((uintptr_t)w & 15) || (p->K % TC_BK)) return cudaErrorInvalidValue;
        cuuint64_t wd[2] = {(cuuint64_t)p->K, (cuuint64_t)n_rows_w};
        cuuint64_t ws[1] = {(cuuint64_t)ldw * 2};
        cuuint32_t wb[2] = {TC_BK, TC_BM};
        r = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)w, wd, ws, wb, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    GemmTcParams q = *p;
    q.dense = w ? 1 : 0;
    // 256-output tiles: only with at most 256 tokens per CTA (two accumulators of 256 columns) and a matrix that
    // is a whole number of such tiles
    if (q.m_halves == 2 && (q.t_tile > 256 || (q.NTL * 16) % (2 * TC_BM) != 0)) q.m_halves = 1;
    if (q.m_halves != 2) q.m_halves = 1;
    dim3 grid(q.NTL * 16 / (TC_BM * q.m_halves), (q.T + q.t_tile - 1) / q.t_tile, 1);
    // CTA pairs: whole 256-token operand tiles only, an even number of output tiles, 128-output CTAs
    if (q.cta_pair && (q.m_halves != 1 || (grid.x & 1) || (q.t_tile != 256 && q.t_tile != 512) || q.T % q.t_tile != 0)) q.cta_pair = 0;
    size_t per_stage = (size_t)q.m_halves * TC_A_BYTES + (size_t)((q.t_tile + 63) / 64) * 64 * 128 / (q.cta_pair ? 2 : 1);
    // as many stages as shared memory holds next to the weight ring, an even number (the two producer
    // groups alternate stages); deep pipelines matter most for few tokens, where a stage is consumed quickly
    const int ring = TC_RING_OF(q.cta_pair != 0);
    const size_t fixed = 1024 + 256 + (size_t)ring * 2 * (TC_PRODUCERS * 32) * 16;
    int stages = (int)((227 * 1024 - fixed) / per_stage);
    stages = stages > 8 ? 8 : stages;
    q.stages = stages < 2 ? 2 : (q.m_halves == 2 ? stages : (stages & ~1));
    size_t smem = b2_gemm_tc_smem(q.cta_pair ? q.t_tile / 2 : q.t_tile, q.stages, q.m_halves, ring);
    static SmemOptIn optin;
    {
        cudaError_t e = optin.ensure(gemm_int4_tc_kernel<false>, smem);
        if (e != cudaSuccess) return e;
    }
    int ks = (q.epi == TC_EPI_RESID_F32 && q.k_splits > 1) ? q.k_splits : 1;
    if (ks > q.KB) ks = q.KB;
    if (ks > 1) { const int per = (q.KB + ks - 1) / ks; ks = (q.KB + per - 1) / per; }     // no empty split
    grid.z = ks;
    if (q.cta_pair) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid; cfg.blockDim = dim3(TC_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        static SmemOptIn optin_pair;
        if (cudaError_t e = optin_pair.ensure(gemm_int4_tc_kernel<true>, smem)) return e;
        return cudaLaunchKernelEx(&cfg, gemm_int4_tc_kernel<true>, q, map, wmap);
    }
    gemm_int4_tc_kernel<false><<<grid, TC_THREADS, smem, stream>>>(q, map, wmap);
    return cudaGetLastError();
}
B2_API int b2_gemm_int4_tc(const GemmTcParams* p, const void* x, int ldx, cudaStream_t stream) {
    return launch_tc(p, nullptr, 0, 0, x, ldx, stream);
}
// Dense fp16 weights w[N][ldw] (row = output feature) take the same pipeline: the weight tile is a
// second TMA load into the stage the dequantising warps would have filled.  p->K, T, t_tile, n_valid (= N),
// ldo, epi, out, status are used; the INT4 fields are ignored.
B2_API int b2_gemm_f16_tc(const GemmTcParams* p, const void* w, int ldw, const void* x, int ldx, cudaStream_t stream) {
    if (!w || p->n_valid < 1) return cudaErrorInvalidValue;
    GemmTcParams q = *p;
    q.KB = q.K / TC_BK;
    q.NTL = (q.n_valid + TC_BM - 1) / TC_BM * (TC_BM / 16);
    q.qfrag = nullptr; q.szfrag = nullptr;
    return launch_tc(&q, w, ldw, q.n_valid, x, ldx, stream);
}
B2_API int b2_sizeof_gemm_tc_params() { return (int)sizeof(GemmTcParams); }
