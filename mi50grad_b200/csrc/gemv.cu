// Decode-path matrix-vector kernels (1..8 token rows) for sm_100a.
//
// gemv_int4: weight-only INT4 (group-wise scale and zero) times fp16
// activations, fp32 accumulation.  It replaces the reference's whole family of
// INT4 GEMV kernels (reference: src/kernels/gemv_int4_v2.hip ... gemv_int4_v8.hip,
// gemv_int4_v5_awq.hip, gemv_int4_dual.hip, gemv_int4_dual_awq.hip,
// gemv_int4_qkv_fused.hip) and the fused communication kernels
// (reference: src/kernels/gemv_int4_p2p_allreduce_rmsnorm.hip,
// kernel_p2p_allreduce_rmsnorm*.hip) with one kernel and four epilogues.
//
// Design, B200-first:
//  * Weights are re-packed once at load time into tensor-core fragment order:
//    a warp's 512-byte load is a [16 outputs x 64 k] tile whose nibbles already
//    sit where mma.m16n8k16 wants them, so decode costs two logic ops per four
//    weights: (w & 0x000f000f) | 0x6400 reads nibble pairs as the fp16 numbers
//    1024+q, and (w & 0x00f000f0) | 0x6400 as 1024+16q.  The second form
//    multiplies activations pre-scaled by 1/16.  Nothing is subtracted per
//    weight: the tensor core accumulates sum((1024+q)*x) in fp32 and the bias
//    1024*sum(x) + zero*sum(x) is removed once per quantisation group.
//  * With 6.5 TB/s of HBM per 148 SMs an SM has ~30 issue slots per 512 bytes,
//    which rules out per-weight SIMT arithmetic; the tensor core is used as an
//    fp32-accumulating dot-product engine, the token rows ride in the 8-wide n
//    dimension of the MMA.
//  * Split-K inside the CTA (4 warps) and across CTAs (deterministic scratch +
//    last-arriver reduction, no atomics on data).
//  * EPI_FINISH: the CTA that completes the last tile publishes this rank's
//    partial sums, signals its peers with st.release.sys, waits (bounded) for
//    theirs, reads the peers' partials over NVLink (plain peer loads or one
//    multimem.ld_reduce), adds the residual and applies the next RMSNorm.  It
//    writes both the updated residual stream and the normalised vector.
#include <cooperative_groups.h>
#include <cstdlib>
#include "gemv.cuh"
namespace cg = cooperative_groups;

#define GEMV_THREADS 256
#define GEMV_WN 2            // warps along n
#define GEMV_WK 4            // warps along k
#define GEMV_NT 4            // 16-wide n-tiles per warp
#define GEMV_STAGE_UN 3         // activation items per thread whose loads are in flight together
#define GEMV_TILE_N (GEMV_WN * GEMV_NT * 16)   // 128
#define GEMV_STAGES 4        // cp.async ring depth per warp (k64-blocks in flight)

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t nib_lo(uint32_t w) {      // halves: 1024 + q
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(r) : "r"(w));
    return r;
}
__device__ __forceinline__ uint32_t nib_hi(uint32_t w) {      // halves: 1024 + 16 q
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(r) : "r"(w));
    return r;
}

// ---------------------------------------------------------------------------
// Tile completion shared by the INT4 and fp16 kernels.  `ybuf` holds the CTA's
// [B2_MAX_ROWS][128] fp32 tile (this CTA's K-slice only when k_splits > 1).
// ---------------------------------------------------------------------------
struct TileCtx {
    int rows, n0, n_pad;     // token rows, first output column, padded N (scratch stride)
    int k_splits;
    int cluster;             // split-K partners are one cluster: reduce through distributed shared memory
    float* scratch;
    int* counters;
    uint32_t tag;            // != 0: tagged hand-off of the split-K partials (see GemvInt4Params::tag_word)
};

#define GEMV_TAG_POLLS (1 << 20)     // polls of one batch of partners before the merge gives up

__device__ void finish_rows(const GemvEpi& e, const CommCtx& c, int rows, uint32_t epoch_next,
                            float* red);

// h_pre / has_pre: the residual of (row 0, column n0 + tid), read by the caller while the weights streamed.
__device__ void complete_tile(float* ybuf, const TileCtx& t, const GemvEpi& e, const CommCtx& c,
                              uint32_t epoch_next, float* red, int* s_flag, float h_pre = 0.f, bool has_pre = false) {
    const int tid = threadIdx.x;
    if (t.k_splits > 1 && t.cluster) {
        // ---- split-K inside a thread-block cluster: the partner CTAs' tiles are read straight from
        // their shared memory (same summation order as the scratch path, so the result is identical);
        // no global round trip, no atomic counter, no last-arriver tail
        cg::cluster_group cl = cg::this_cluster();
        cl.sync();
        if (blockIdx.y == 0) {
            for (int i = tid; i < t.rows * GEMV_TILE_N; i += GEMV_THREADS) {
                float v[8];
#pragma unroll
                for (int ks = 1; ks < 8; ++ks) v[ks] = ks < t.k_splits ? cl.map_shared_rank(ybuf, ks)[i] : 0.f;
                float s = ybuf[i];
#pragma unroll
                for (int ks = 1; ks < 8; ++ks) if (ks < t.k_splits) s += v[ks];
                ybuf[i] = s;
            }
        }
        cl.sync();                                   // partners may exit (their shared memory is no longer read)
        if (blockIdx.y != 0) return;
        __syncthreads();
    } else
    // ---- cross-CTA split-K, tagged: slices 1.. store {value, tag} pairs and leave; slice 0 polls them and
    // sums in the order of the slices (the same order, and therefore the same bits, as the counter protocol)
    if (t.k_splits > 1 && t.tag) {
        float2* sc = (float2*)t.scratch;
        if (blockIdx.y != 0) {
            for (int i = tid; i < t.rows * GEMV_TILE_N; i += GEMV_THREADS) {
                const int r = i / GEMV_TILE_N, nl = i % GEMV_TILE_N;
                float2 v = make_float2(ybuf[r * GEMV_TILE_N + nl], __uint_as_float(t.tag));
                float2* dst = &sc[((size_t)(blockIdx.y - 1) * t.rows + r) * t.n_pad + t.n0 + nl];
                asm volatile("st.global.v2.f32 [%0], {%1, %2};" :: "l"(dst), "f"(v.x), "f"(v.y) : "memory");
            }
            return;
        }
        bool late = false;
        for (int i = tid; i < t.rows * GEMV_TILE_N; i += GEMV_THREADS) {
            const int r = i / GEMV_TILE_N, nl = i % GEMV_TILE_N;
            float s = ybuf[r * GEMV_TILE_N + nl];
            for (int k0 = 1; k0 < t.k_splits; k0 += 8) {
                float v[8];
                unsigned need = 0;
#pragma unroll
                for (int u = 0; u < 8; ++u) { v[u] = 0.f; if (k0 + u < t.k_splits) need |= 1u << u; }
                for (int it = 0; it < GEMV_TAG_POLLS && need; ++it) {
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        if (need & (1u << u)) {
                            const float2* src = &sc[((size_t)(k0 + u - 1) * t.rows + r) * t.n_pad + t.n0 + nl];
                            float a, b;
                            asm volatile("ld.volatile.global.v2.f32 {%0, %1}, [%2];" : "=f"(a), "=f"(b) : "l"(src) : "memory");
                            if (__float_as_uint(b) == t.tag) { v[u] = a; need &= ~(1u << u); }
                        }
                    }
                }
                if (need) late = true;
#pragma unroll
                for (int u = 0; u < 8; ++u) if (k0 + u < t.k_splits) s += v[u];
            }
            ybuf[r * GEMV_TILE_N + nl] = s;
        }
        if (late && c.status) report_timeout(c, B2_KID_GEMV_SPLITK, (int)blockIdx.x, t.tag);
        __syncthreads();
    } else
    // ---- cross-CTA split-K: publish, count, last arriver sums in a fixed order
    if (t.k_splits > 1) {
        for (int i = tid; i < t.rows * GEMV_TILE_N; i += GEMV_THREADS) {
            int r = i / GEMV_TILE_N, nl = i % GEMV_TILE_N;
            t.scratch[((size_t)blockIdx.y * t.rows + r) * t.n_pad + t.n0 + nl] = ybuf[r * GEMV_TILE_N + nl];
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int old = atomicAdd(&t.counters[blockIdx.x], 1);
            int last = (old == t.k_splits - 1);
            if (last) t.counters[blockIdx.x] = 0;
            *s_flag = last;
            __threadfence();
        }
        __syncthreads();
        if (!*s_flag) return;
        for (int i = tid; i < t.rows * GEMV_TILE_N; i += GEMV_THREADS) {
            int r = i / GEMV_TILE_N, nl = i % GEMV_TILE_N;
            // the pieces of up to eight splits are requested together: a load-then-add loop would pay one
            // trip to L2 per split; the sum keeps the order of the splits
            float s = 0.f;
            for (int k0 = 0; k0 < t.k_splits; k0 += 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    v[u] = (k0 + u < t.k_splits) ? ld_cg_f32(&t.scratch[((size_t)(k0 + u) * t.rows + r) * t.n_pad + t.n0 + nl]) : 0.f;
#pragma unroll
                for (int u = 0; u < 8; ++u) s += v[u];
            }
            ybuf[r * GEMV_TILE_N + nl] = s;
        }
        __syncthreads();
    }
    // ---- epilogues
    if (e.mode == EPI_STORE_F16) {
        __half* out = (__half*)e.out;
        for (int i = tid; i < t.rows * GEMV_TILE_N; i += GEMV_THREADS) {
            int r = i / GEMV_TILE_N, n = t.n0 + i % GEMV_TILE_N;
            if (n < e.n_valid) out[(size_t)r * e.ldo + n] = __float2half(ybuf[i]);
        }
    } else if (e.mode == EPI_STORE_F32) {
        float* out = (float*)e.out;
        for (int i = tid; i < t.rows * GEMV_TILE_N; i += GEMV_THREADS) {
            int r = i / GEMV_TILE_N, n = t.n0 + i % GEMV_TILE_N;
            if (n < e.n_valid) out[(size_t)r * e.ldo + n] = ybuf[i];
        }
    } else if (e.mode == EPI_SILU_PAIR) {
        __half* out = (__half*)e.out;
        for (int i = tid; i < t.rows * (GEMV_TILE_N / 2); i += GEMV_THREADS) {
            int r = i / (GEMV_TILE_N / 2), j = i % (GEMV_TILE_N / 2);
            int base = r * GEMV_TILE_N + (j >> 3) * 16 + (j & 7);
            int o = t.n0 / 2 + j;
            if (o < e.n_valid) out[(size_t)r * e.ldo + o] = __float2half(silu_f(ybuf[base]) * ybuf[base + 8]);
        }
    } else {   // EPI_FINISH
        const bool local = (e.fin_flags & FIN_NO_COMM) || c.tp <= 1;
        const int np = (e.n_valid + GEMV_TILE_N - 1) / GEMV_TILE_N;
        if (local) {
            // No exchange: every tile adds the residual for its own 128 columns and leaves the
            // sum of squares of what it wrote; the consumer applies the RMSNorm lazily.  No
            // counter, no fence, no serial tail.
            for (int r = 0; r < t.rows; ++r) {
                float sq = 0.f;
                if (tid < GEMV_TILE_N) {
                    int n = t.n0 + tid;
                    if (n < e.n_valid) {
                        size_t off = (size_t)r * e.n_valid + n;
                        float v = ybuf[r * GEMV_TILE_N + tid];
                        if (e.fin_flags & FIN_ADD_EXTRA) v += e.extra[off];
                        if (e.fin_flags & FIN_SAVE_EXTRA) e.extra[off] = v;
                        float hv = ((has_pre && r == 0) ? h_pre : e.h[off]) + v;
                        e.hout[off] = hv;
                        sq = hv * hv;
                    }
                }
                float tot = block_sum(sq, red);
                const int snp = e.ss_np > 0 ? e.ss_np : np, per = snp / np;
                if (tid < per) e.ss_part[(size_t)r * snp + blockIdx.x * per + tid] = tid == 0 ? tot : 0.f;
            }
            return;
        }
        float* part = c.part[c.rank] + (size_t)(epoch_next & 1) * c.part_stride;
        for (int i = tid; i < t.rows * GEMV_TILE_N; i += GEMV_THREADS) {
            int r = i / GEMV_TILE_N, n = t.n0 + i % GEMV_TILE_N;
            if (n < e.n_valid) {
                float v = ybuf[i];
                if (e.fin_flags & FIN_ADD_EXTRA) v += e.extra[(size_t)r * e.n_valid + n];
                part[(size_t)r * e.n_valid + n] = v;
            }
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int old = atomicAdd(&t.counters[gridDim.x], 1);
            int last = (old == (int)gridDim.x - 1);
            if (last) t.counters[gridDim.x] = 0;
            *s_flag = last;
            __threadfence();
        }
        __syncthreads();
        if (!*s_flag) return;
        finish_rows(e, c, t.rows, epoch_next, red);
    }
}

// One CTA: exchange the ranks' partial sums over NVLink, add the residual, leave the sum
// of squares for the consumer's lazy RMSNorm (and, if asked, the normalised vector).
// n_valid <= 8192.
__device__ void finish_rows(const GemvEpi& e, const CommCtx& c, int rows, uint32_t epoch_next,
                            float* red) {
    const int tid = threadIdx.x;
    const int H = e.n_valid;
    const int np = (H + GEMV_TILE_N - 1) / GEMV_TILE_N;
    __shared__ int s_fail;
    if (tid == 0) s_fail = 0;
    if (tid == 0 && c.trace) c.trace[0] = globaltimer_ns();
    __syncthreads();
    if (tid == 0) *c.epoch = epoch_next;
    if (tid < c.tp && tid != c.rank && !(e.fin_flags & FIN_TEST_WITHHOLD_SIGNAL))
        st_release_sys_u32(c.sig[tid] + c.rank, epoch_next);
    if (tid < c.tp && tid != c.rank) {
        if (!wait_reached(c.sig[c.rank] + tid, epoch_next, c.wait_ns)) {
            report_timeout(c, B2_KID_GEMV_FIN, tid, epoch_next);
            s_fail = 1;
        }
    }
    __syncthreads();
    if (tid == 0 && c.trace) c.trace[1] = globaltimer_ns();
    const bool exchange = !s_fail;
    const size_t poff = (size_t)(epoch_next & 1) * c.part_stride;
    const float* mine = c.part[c.rank] + poff;
    const float* peer[B2_MAX_TP];
#pragma unroll
    for (int pr = 0; pr < B2_MAX_TP; ++pr) peer[pr] = c.part[pr < c.tp ? pr : 0] + poff;
    for (int r = 0; r < rows; ++r) {
        // all loads of a row are issued before anything is stored, so the NVLink round trips overlap
        float4 hv[8], yv[8];
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            int n = (it * GEMV_THREADS + tid) * 4;
            if (n < H) {
                size_t off = (size_t)r * H + n;
                if (exchange && c.mc_part) {
                    yv[it] = multimem_ld_reduce_v4(c.mc_part + poff + off);
                } else if (exchange) {
                    float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int pr = 0; pr < B2_MAX_TP; ++pr) {
                        if (pr < c.tp) {
                            float4 v = ld_relaxed_sys_v4(peer[pr] + off);
                            y.x += v.x; y.y += v.y; y.z += v.z; y.w += v.w;
                        }
                    }
                    yv[it] = y;
                } else {
                    yv[it] = ld_cg_v4(mine + off);
                }
                hv[it] = *(const float4*)(e.h + off);
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            int n = (it * GEMV_THREADS + tid) * 4;
            if (n < H) {
                size_t off = (size_t)r * H + n;
                float4 h = hv[it];
                h.x += yv[it].x; h.y += yv[it].y; h.z += yv[it].z; h.w += yv[it].w;
                *(float4*)(e.hout + off) = h;
                hv[it] = h;
                ss += h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
            }
        }
        float tot = block_sum(ss, red);
        if (tid == 0 && c.trace) c.trace[2] = globaltimer_ns();
        const int snp = e.ss_np > 0 ? e.ss_np : np;
        for (int i = tid; i < snp; i += GEMV_THREADS) e.ss_part[(size_t)r * snp + i] = (i == 0) ? tot : 0.f;
        if (e.xn == nullptr || (e.fin_flags & FIN_NO_NORM)) continue;
        float inv = rsqrtf(tot / (float)H + e.eps);
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            int n = (it * GEMV_THREADS + tid) * 4;
            if (n < H) {
                const __half2* w2 = (const __half2*)(e.norm_w + n);
                float2 w01 = __half22float2(w2[0]), w23 = __half22float2(w2[1]);
                __half2 o0 = __floats2half2_rn(hv[it].x * inv * w01.x, hv[it].y * inv * w01.y);
                __half2 o1 = __floats2half2_rn(hv[it].z * inv * w23.x, hv[it].w * inv * w23.y);
                __half2* dst = (__half2*)(e.xn + (size_t)r * H + n);
                dst[0] = o0;
                dst[1] = o1;
            }
        }
    }
}

// One warp's share of the L2 prefetch for the next INT4 GEMV of the stream: the streams (CTA, warp) of that
// launch are dealt round-robin to the warps of this one; lane 0 asks L2 for the first blocks of each.
__device__ __forceinline__ void prefetch_next_weights(const GemvInt4Params& p, int warp, int lane) {
    if (lane != 0) return;
    const int my = ((int)blockIdx.y * (int)gridDim.x + (int)blockIdx.x) * (GEMV_THREADS / 32) + warp;
    const int n_mine = (int)(gridDim.x * gridDim.y) * (GEMV_THREADS / 32);
    if (p.pf_span) {
        // a contiguous span, one slice per warp of this launch
        const long long per = ((p.pf_span_bytes + n_mine - 1) / n_mine + 15) & ~15ll;
        const long long off = per * my;
        if (off < p.pf_span_bytes) {
            const uint32_t bytes = (uint32_t)min(per, (p.pf_span_bytes - off) & ~15ll);
            if (bytes) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"((const char*)p.pf_span + off), "r"(bytes) : "memory");
        }
    }
    if (!p.pf_q) return;
    const int n_next = p.pf_nx * p.pf_ks * (GEMV_THREADS / 32);
    for (int sid = my; sid < n_next; sid += n_mine) {
        const int cta = sid / (GEMV_THREADS / 32), w = sid % (GEMV_THREADS / 32);
        const int x = cta % p.pf_nx, y = cta / p.pf_nx;
        const int wn = w % GEMV_WN, wk = w / GEMV_WN;
        const int b0 = y * (GEMV_WK * p.pf_L) + wk * p.pf_L;
        const int b1 = min(min(p.pf_KB, (y + 1) * (GEMV_WK * p.pf_L)), b0 + p.pf_L);
        const int nb = min(b1 - b0, p.pf_blocks);
        if (nb <= 0) continue;
        const uint4* src = p.pf_q + ((size_t)(x * GEMV_WN + wn) * p.pf_KB + b0) * (GEMV_NT * 32);
        const uint32_t bytes = (uint32_t)nb * (GEMV_NT * 32 * 16);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(src), "r"(bytes) : "memory");
    }
}

// ---------------------------------------------------------------------------
// INT4 kernel
// ---------------------------------------------------------------------------
template <bool FAST>
__global__ void __launch_bounds__(GEMV_THREADS, 2) gemv_int4_kernel(const GemvInt4Params p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wn = warp % GEMV_WN, wk = warp / GEMV_WN;
    const int g = lane >> 2, t = lane & 3;
    const int M = p.rows;
    const int maxCh = 2 * GEMV_WK * p.L;
    const int cta_b0 = blockIdx.y * (GEMV_WK * p.L);
    const int cta_b1 = min(p.KB, cta_b0 + GEMV_WK * p.L);
    const int nCh = max(0, cta_b1 - cta_b0) * 2;
    pdl_launch_dependents();

    uint4* xf = (uint4*)smem;                                        // [maxCh][M][4] (+1 zero entry)
    float2* cs = (float2*)(smem + ((size_t)maxCh * M * 4 + 4) * 16); // [maxCh][8]
    float* redbuf = (float*)((unsigned char*)cs + (size_t)maxCh * 8 * 8);   // [WK*WN*NT*128]
    float* ybuf = redbuf + GEMV_WK * GEMV_WN * GEMV_NT * 128;        // [8][128]
    float* red32 = ybuf + B2_MAX_ROWS * GEMV_TILE_N;                 // [32]
    int* s_flag = (int*)(red32 + 32);          // 4 ints, then the weight ring (16-byte aligned)

    // ---- this warp owns GEMV_NT n-tiles (contiguous in memory per k-block) over blocks [wb0, wb1).
    // Weights stream through a per-warp cp.async ring: GEMV_STAGES-1 blocks of 2 KB are in
    // flight per warp at all times (each lane copies and later reads only its own 16 bytes,
    // so no cross-lane synchronisation).  The ring is primed before anything else so that
    // HBM is busy while the activations are staged.
    const int wt = blockIdx.x * GEMV_WN + wn;
    const int wb0 = cta_b0 + wk * p.L, wb1 = min(cta_b1, wb0 + p.L);
    const int nb = max(0, wb1 - wb0);
    uint4* rp = (uint4*)(s_flag + 4) + (size_t)warp * (GEMV_STAGES * GEMV_NT * 32) + lane;
    const uint4* gp = p.qfrag + ((size_t)wt * p.KB + wb0) * (GEMV_NT * 32) + lane;
    // FAST: the 256 bytes of scale/zero pairs of a group ride along with the group's first weight block, so
    // that nothing in the main loop waits on a global load
    uint4* szr = (uint4*)(s_flag + 4) + (size_t)(GEMV_THREADS / 32) * (GEMV_STAGES * GEMV_NT * 32) + (size_t)warp * (GEMV_STAGES * 16);
    const uint4* szg = (const uint4*)(p.szfrag + (size_t)wt * p.G * (GEMV_NT * 8));      // 16 uint4 per group
#pragma unroll
    for (int s = 0; s < GEMV_STAGES - 1; ++s) {
        if (s < nb) {
#pragma unroll
            for (int i = 0; i < GEMV_NT; ++i) cp_async16(rp + (s * GEMV_NT + i) * 32, gp + (s * GEMV_NT + i) * 32);
            // slot of a group's pairs: the group's index inside this warp's slice, modulo the ring depth (blocks
            // b .. b+3 in flight touch at most three groups, so a slot is free again before it is reused)
            if (FAST && !(s & 1) && lane < 16) cp_async16(szr + ((s >> 1) & (GEMV_STAGES - 1)) * 16 + lane, szg + (size_t)((wb0 + s) >> 1) * 16 + lane);
        }
        cp_async_commit();
    }
    gp += (GEMV_STAGES - 1) * GEMV_NT * 32;    // next block to prefetch
    if (nb <= GEMV_STAGES - 1) prefetch_next_weights(p, warp, lane);      // all of this warp's weights are requested
    // Weights do not depend on earlier kernels; everything below does.
    pdl_wait();
    const uint32_t epoch_next = (p.epi.mode == EPI_FINISH && p.comm.tp > 1) ? (*p.comm.epoch + 1u) : 0u;
    if (p.comm.trace && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) p.comm.trace[3] = globaltimer_ns();

    // tag of this launch's split-K pairs (requested now, used at the very end)
    const uint32_t tag = (p.tag_word && p.k_splits > 1) ? (*p.tag_word + (uint32_t)p.tag_base) : 0u;
    // the residual this tile's epilogue adds (one token row, no exchange): requested now, used at the very end
    float h_pre = 0.f;
    bool has_pre = false;
    if (p.epi.mode == EPI_FINISH && M == 1 && ((p.epi.fin_flags & FIN_NO_COMM) || p.comm.tp <= 1) && tid < GEMV_TILE_N) {
        const int n = blockIdx.x * GEMV_TILE_N + tid;
        if (n < p.epi.n_valid) { h_pre = p.epi.h[n]; has_pre = true; }
    }

    // ---- stage activations in MMA B-fragment order, with per-chunk bias sums
    for (int i = tid; i < nCh * 8; i += GEMV_THREADS)
        if ((i & 7) >= M) cs[i] = make_float2(0.f, 0.f);
    if (tid < 4) xf[(size_t)maxCh * M * 4 + tid] = make_uint4(0u, 0u, 0u, 0u);
    const int items = nCh * 4;
    float* s_inv = red32;                       // [rows] 1/rms per row when the input is lazy-normed
    // Loads first, arithmetic after: the inputs of up to GEMV_STAGE_UN items per thread (and, under them, the
    // partial sums of squares of the lazy RMSNorm) are requested before anything waits on one of them, so
    // staging costs one trip to L2 instead of one per item.
    bool inv_ready = !p.ln.h;
    for (int m = 0; m < M; ++m) {
        const __half* xr = p.x + (size_t)m * p.ldx;
        const float* hr = p.ln.h ? p.ln.h + (size_t)m * p.ln.H : nullptr;
        for (int base0 = 0; base0 < items; base0 += GEMV_STAGE_UN * GEMV_THREADS) {
            float2 hv[GEMV_STAGE_UN][4];
            __half2 wv[GEMV_STAGE_UN][4];
#pragma unroll
            for (int u = 0; u < GEMV_STAGE_UN; ++u) {
                const int item = base0 + u * GEMV_THREADS + tid;
                const bool valid = item < items;
                const int k0 = (cta_b0 * 2 + (item >> 2)) * 32 + 2 * (item & 3);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int k = k0 + 8 * q;
                    hv[u][q] = make_float2(0.f, 0.f);
                    wv[u][q] = __float2half2_rn(0.f);
                    if (valid && k < p.K) {
                        if (hr) { hv[u][q] = *(const float2*)(hr + k); wv[u][q] = *(const __half2*)(p.ln.w + k); }
                        else wv[u][q] = *(const __half2*)(xr + k);
                    }
                }
            }
            if (!inv_ready) {
                if (warp < M) { float v = lazy_inv_rms(p.ln, warp, lane); if (lane == 0) s_inv[warp] = v; }
                __syncthreads();
                inv_ready = true;
            }
            const float inv = hr ? s_inv[m] : 0.f;
#pragma unroll
            for (int u = 0; u < GEMV_STAGE_UN; ++u) {
                const int item = base0 + u * GEMV_THREADS + tid;
                if (base0 + u * GEMV_THREADS >= items) break;          // uniform: no thread has an item here
                const bool valid = item < items;
                const int tt = item & 3, cl = item >> 2;
                __half2 a0, a1, b0, b1;
                if (hr) {
                    auto nrm = [&](int q) -> __half2 {
                        const float2 w = __half22float2(wv[u][q]);
                        return __floats2half2_rn(hv[u][q].x * inv * w.x, hv[u][q].y * inv * w.y);
                    };
                    a0 = nrm(0); a1 = nrm(1); b0 = nrm(2); b1 = nrm(3);
                } else {
                    a0 = wv[u][0]; a1 = wv[u][1]; b0 = wv[u][2]; b1 = wv[u][3];
                }
                const __half2 sixteenth = __float2half2_rn(0.0625f);
                b0 = __hmul2(b0, sixteenth);
                b1 = __hmul2(b1, sixteenth);
                float2 fa0 = __half22float2(a0), fa1 = __half22float2(a1);
                float2 fb0 = __half22float2(b0), fb1 = __half22float2(b1);
                float sa = fa0.x + fa0.y + fa1.x + fa1.y;
                float sb = fb0.x + fb0.y + fb1.x + fb1.y;
                sa += __shfl_xor_sync(0xffffffffu, sa, 1);
                sb += __shfl_xor_sync(0xffffffffu, sb, 1);
                sa += __shfl_xor_sync(0xffffffffu, sa, 2);
                sb += __shfl_xor_sync(0xffffffffu, sb, 2);
                if (valid) {
                    uint4 v;
                    v.x = *(uint32_t*)&a0; v.y = *(uint32_t*)&a1; v.z = *(uint32_t*)&b0; v.w = *(uint32_t*)&b1;
                    xf[(cl * M + m) * 4 + tt] = v;
                    if (tt == 0) cs[cl * 8 + m] = make_float2(1024.f * (sa + sb), sa + 16.f * sb);
                }
            }
        }
    }
    if (!inv_ready) __syncthreads();               // (no items at all: keep the barrier count uniform)
    __syncthreads();

    float acc[GEMV_NT][4], tot[GEMV_NT][4];
#pragma unroll
    for (int i = 0; i < GEMV_NT; ++i)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[i][r] = tot[i][r] = 0.f;
    float c1r0 = 0.f, c1r1 = 0.f, c2r0 = 0.f, c2r1 = 0.f;
    int cur = -1;
    const uint2* szp = p.szfrag + (size_t)wt * p.G * (GEMV_NT * 8) + g;

    int sz_stage = 0;                          // FAST: ring stage that holds the scale/zero pairs of the group being flushed
    auto flush = [&](int grp) {
#pragma unroll
        for (int i = 0; i < GEMV_NT; ++i) {
            uint2 sz = FAST ? ((const uint2*)(szr + sz_stage * 16))[i * 8 + g] : ldg_nc_v2(szp + ((size_t)grp * GEMV_NT + i) * 8);
            float2 s = __half22float2(*(__half2*)&sz.x), z = __half22float2(*(__half2*)&sz.y);
            tot[i][0] += s.x * (acc[i][0] - c1r0 - z.x * c2r0);
            tot[i][1] += s.x * (acc[i][1] - c1r1 - z.x * c2r1);
            tot[i][2] += s.y * (acc[i][2] - c1r0 - z.y * c2r0);
            tot[i][3] += s.y * (acc[i][3] - c1r1 - z.y * c2r1);
            acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        }
        c1r0 = c1r1 = c2r0 = c2r1 = 0.f;
    };

    // per-lane activation pointer: lanes whose token row does not exist read a zero entry with stride 0
    const int cl0 = 2 * (wb0 - cta_b0);
    const uint4* xp = (g < M) ? xf + ((size_t)cl0 * M + g) * 4 + t : xf + (size_t)maxCh * M * 4 + t;
    const int xstride = (g < M) ? M * 4 : 0;
    const float4* cp4 = (const float4*)(cs + (size_t)cl0 * 8 + 2 * t);

    for (int bb = 0; bb < nb; bb += GEMV_STAGES) {
#pragma unroll
        for (int s = 0; s < GEMV_STAGES; ++s) {
            const int br = bb + s;
            if (br < nb) {
                if (br + GEMV_STAGES - 1 < nb) {
#pragma unroll
                    for (int i = 0; i < GEMV_NT; ++i)
                        cp_async16(rp + (((s + GEMV_STAGES - 1) % GEMV_STAGES) * GEMV_NT + i) * 32, gp + i * 32);
                    gp += GEMV_NT * 32;
                    if (br + GEMV_STAGES == nb) prefetch_next_weights(p, warp, lane);     // that was this warp's last block
                    // block br + 3 is the first of its group exactly when s is odd (the slice starts on an even block)
                    if (FAST && (s & 1) && lane < 16)
                        cp_async16(szr + (((br + GEMV_STAGES - 1) >> 1) & (GEMV_STAGES - 1)) * 16 + lane,
                                   szg + (size_t)((wb0 + br + GEMV_STAGES - 1) >> 1) * 16 + lane);
                }
                cp_async_commit();
                cp_async_wait<GEMV_STAGES - 1>();
                uint4 w[GEMV_NT];
#pragma unroll
                for (int i = 0; i < GEMV_NT; ++i) w[i] = rp[(s * GEMV_NT + i) * 32];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    if (!FAST) {
                        const int grp = (2 * (wb0 + br) + j + p.off32) >> p.gshift;
                        if (grp != cur) {
                            if (cur >= 0) flush(cur);
                            cur = grp;
                        }
                    }
                    const uint4 xv = *xp;
                    xp += xstride;
                    const float4 cv = cp4[j * 4];
                    c1r0 += cv.x; c2r0 += cv.y; c1r1 += cv.z; c2r1 += cv.w;
#pragma unroll
                    for (int i = 0; i < GEMV_NT; ++i) {
                        uint32_t w0 = j ? w[i].z : w[i].x, w1 = j ? w[i].w : w[i].y;
                        uint32_t w0s = w0 >> 8, w1s = w1 >> 8;
                        mma16816(acc[i], nib_lo(w0), nib_lo(w0s), nib_lo(w1), nib_lo(w1s), xv.x, xv.y);
                        mma16816(acc[i], nib_hi(w0), nib_hi(w0s), nib_hi(w1), nib_hi(w1s), xv.z, xv.w);
                    }
                }
                cp4 += 8;
                // FAST: groups of 128 k aligned to even blocks, so a group ends after every odd block
                if (FAST && (s & 1)) { sz_stage = (br >> 1) & (GEMV_STAGES - 1); flush((wb0 + br) >> 1); }
            }
        }
    }
    cp_async_wait<0>();
    if (FAST) { if (nb & 1) { sz_stage = ((nb - 1) >> 1) & (GEMV_STAGES - 1); flush((wb0 + nb - 1) >> 1); } }
    else if (cur >= 0) flush(cur);

    // ---- in-CTA reduction over the k-warps into ybuf[row][n_local]
#pragma unroll
    for (int i = 0; i < GEMV_NT; ++i)
        *(float4*)&redbuf[(((wk * GEMV_WN + wn) * GEMV_NT + i) * 32 + lane) * 4] =
            make_float4(tot[i][0], tot[i][1], tot[i][2], tot[i][3]);
    __syncthreads();
    for (int e = tid; e < GEMV_WN * GEMV_NT * 128; e += GEMV_THREADS) {
        int wne = e / (GEMV_NT * 128), rem = e % (GEMV_NT * 128);
        int i = rem >> 7, ln = (rem >> 2) & 31, r = rem & 3;
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < GEMV_WK; ++k) s += redbuf[((k * GEMV_WN + wne) * GEMV_NT + i) * 128 + (rem & 127)];
        int nl = wne * GEMV_NT * 16 + i * 16 + (ln >> 2) + 8 * (r >> 1);
        int row = 2 * (ln & 3) + (r & 1);
        ybuf[row * GEMV_TILE_N + nl] = s;
    }
    __syncthreads();

    TileCtx tc;
    tc.rows = M; tc.n0 = blockIdx.x * GEMV_TILE_N; tc.n_pad = p.NTL * 16;
    tc.k_splits = p.k_splits; tc.scratch = p.scratch; tc.counters = p.counters; tc.cluster = p.cluster_splitk;
    tc.tag = tag;
    complete_tile(ybuf, tc, p.epi, p.comm, epoch_next, red32, s_flag, h_pre, has_pre);
}

// ---------------------------------------------------------------------------
// fp16-weight kernel (lm_head, fp16-attention checkpoints).  Replaces the
// reference's gemv_fp16_v2 (reference: src/kernels/gemv_fp16_v2.hip:22-88).
// CTA tile: 128 outputs x kslice; each warp owns 16 outputs, 4 at a time.
// ---------------------------------------------------------------------------
template <int MR>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_f16_kernel(const GemvF16Params p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int M = p.rows;
    const int k0 = blockIdx.y * p.kslice;
    const int klen = min(p.kslice, p.K - k0);
    pdl_launch_dependents();
    __half* xs = (__half*)smem;                                      // [MR][kslice]
    float* ybuf = (float*)(smem + (size_t)MR * p.kslice * 2);        // [8][128]
    float* red32 = ybuf + B2_MAX_ROWS * GEMV_TILE_N;
    int* s_flag = (int*)(red32 + 32);
    const uint32_t epoch_next = (p.epi.mode == EPI_FINISH && p.comm.tp > 1) ? (*p.comm.epoch + 1u) : 0u;

    // stage the activations (normalised on the way when the input is the lazy fp32 stream): the loads of up
    // to GEMV_STAGE_UN pieces per thread, and under them the partial sums of the norm, are requested before
    // anything waits on one of them
    bool inv_ready = !p.ln.h;
    for (int i0 = tid * 8; i0 < MR * p.kslice; i0 += GEMV_STAGE_UN * GEMV_THREADS * 8) {
        uint4 raw[GEMV_STAGE_UN];
        float2 hv[GEMV_STAGE_UN][4];
#pragma unroll
        for (int u = 0; u < GEMV_STAGE_UN; ++u) {
            const int i = i0 + u * GEMV_THREADS * 8;
            const int m = i / p.kslice, kk = i % p.kslice;
            raw[u] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int q = 0; q < 4; ++q) hv[u][q] = make_float2(0.f, 0.f);
            if (i < MR * p.kslice && m < M && kk < klen) {
                if (p.ln.h) {
                    const float* hr = p.ln.h + (size_t)m * p.ln.H + k0 + kk;
                    raw[u] = *(const uint4*)(p.ln.w + k0 + kk);
#pragma unroll
                    for (int q = 0; q < 4; ++q) hv[u][q] = *(const float2*)(hr + 2 * q);
                } else {
                    raw[u] = *(const uint4*)(p.x + (size_t)m * p.ldx + k0 + kk);
                }
            }
        }
        if (!inv_ready) {
            if (warp < M) { float v = lazy_inv_rms(p.ln, warp, lane); if (lane == 0) red32[warp] = v; }
            __syncthreads();
            inv_ready = true;
        }
#pragma unroll
        for (int u = 0; u < GEMV_STAGE_UN; ++u) {
            const int i = i0 + u * GEMV_THREADS * 8;
            if (i >= MR * p.kslice) break;
            const int m = i / p.kslice;
            uint4 v = raw[u];
            if (p.ln.h) {
                const float inv = m < M ? red32[m] : 0.f;
                const __half2* wv = (const __half2*)&raw[u];
                __half2* o = (__half2*)&v;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 ww = __half22float2(wv[q]);
                    o[q] = __floats2half2_rn(hv[u][q].x * inv * ww.x, hv[u][q].y * inv * ww.y);
                }
            }
            *(uint4*)(xs + i) = v;
        }
    }
    if (!inv_ready) __syncthreads();
    for (int i = tid; i < B2_MAX_ROWS * GEMV_TILE_N; i += GEMV_THREADS) ybuf[i] = 0.f;
    __syncthreads();

    const int n_base = blockIdx.x * GEMV_TILE_N + warp * 16;
#pragma unroll 1
    for (int rb = 0; rb < 16; rb += 4) {
        float acc[4][MR];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int m = 0; m < MR; ++m) acc[r][m] = 0.f;
        const __half* wr[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            int n = min(n_base + rb + r, p.N - 1);
            wr[r] = p.w + (size_t)n * p.ldw + k0;
        }
        for (int kk = lane * 8; kk < klen; kk += 256) {
            uint4 wv[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) wv[r] = ldg_nc_v4(wr[r] + kk);
#pragma unroll
            for (int m = 0; m < MR; ++m) {
                uint4 xv = *(const uint4*)(xs + m * p.kslice + kk);
                const __half2* x2 = (const __half2*)&xv;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const __half2* w2 = (const __half2*)&wv[r];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float2 a = __half22float2(w2[q]), b = __half22float2(x2[q]);
                        acc[r][m] = fmaf(a.x, b.x, acc[r][m]);
                        acc[r][m] = fmaf(a.y, b.y, acc[r][m]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int m = 0; m < MR; ++m) {
                float v = warp_sum(acc[r][m]);
                if (lane == 0 && m < M) ybuf[m * GEMV_TILE_N + warp * 16 + rb + r] = v;
            }
    }
    __syncthreads();
    TileCtx tc;
    tc.rows = M; tc.n0 = blockIdx.x * GEMV_TILE_N; tc.n_pad = (int)gridDim.x * GEMV_TILE_N;
    tc.k_splits = p.k_splits; tc.scratch = p.scratch; tc.counters = p.counters;
    tc.cluster = 0; tc.tag = 0;
    complete_tile(ybuf, tc, p.epi, p.comm, epoch_next, red32, s_flag);
}

// ---------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------
B2_API size_t b2_gemv_int4_smem(int rows, int L) {
    size_t maxCh = 2 * GEMV_WK * (size_t)L;
    return (maxCh * rows + 1) * 64 + maxCh * 64 + (GEMV_WK * GEMV_WN * GEMV_NT * 128 + B2_MAX_ROWS * GEMV_TILE_N + 32 + 4) * 4
           + (size_t)(GEMV_THREADS / 32) * GEMV_STAGES * (GEMV_NT * 512 + 256);
}

B2_API int b2_gemv_int4(const GemvInt4Params* p, cudaStream_t stream) {
    if (p->rows < 1 || p->rows > B2_MAX_ROWS) return cudaErrorInvalidValue;
    if (p->epi.mode == EPI_FINISH && p->epi.n_valid > 8192) return cudaErrorInvalidValue;
    size_t smem = b2_gemv_int4_smem(p->rows, p->L);
    // groups of 128 aligned to even k-blocks let the kernel drop all per-chunk group bookkeeping
    const bool fast = p->gshift == 2 && p->off32 == 0 && (p->L % 2 == 0);
    static SmemOptIn optin[2];
    {
        cudaError_t e = fast ? optin[1].ensure(gemv_int4_kernel<true>, smem) : optin[0].ensure(gemv_int4_kernel<false>, smem);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p->NTL * 16 / GEMV_TILE_N, p->k_splits);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    GemvInt4Params q = *p;
    q.cluster_splitk = 0;
    if (q.tag_word && q.k_splits > 1) {
        // the tagged hand-off makes one CTA wait for others of the same grid: only with the whole grid resident
        static std::mutex occ_mu;
        static int sms = 0, n_cached = 0;
        static size_t cached_smem[64];
        static int cached_fast[64], cached_per_sm[64];
        int per_sm = 0;
        {
            std::lock_guard<std::mutex> lock(occ_mu);
            if (!sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
            for (int i = 0; i < n_cached; ++i)
                if (cached_smem[i] == smem && cached_fast[i] == (int)fast) per_sm = cached_per_sm[i];
            if (!per_sm) {
                int n = 0;
                cudaError_t e = fast ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemv_int4_kernel<true>, GEMV_THREADS, smem)
                                     : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemv_int4_kernel<false>, GEMV_THREADS, smem);
                per_sm = (e == cudaSuccess && n > 0) ? n : -1;
                if (n_cached < 64) { cached_smem[n_cached] = smem; cached_fast[n_cached] = (int)fast; cached_per_sm[n_cached++] = per_sm; }
            }
        }
        if (per_sm < 0 || (long long)cfg.gridDim.x * cfg.gridDim.y > (long long)sms * per_sm) q.tag_word = nullptr;
    }
    // Optional: the split-K partners of an output tile as one cluster along grid y, reducing through
    // distributed shared memory.  Measured slower than the scratch + counter path on B200 (down
    // projection 21.0 us against 14.7 us, decode 180.5 against 188.4 tok/s: clusters of 7 CTAs are
    // placed with less freedom), so it is off unless B200GRAD_CLUSTER_SPLITK is set.
    static const bool want_cluster = getenv("B200GRAD_CLUSTER_SPLITK") != nullptr;
    if (want_cluster && p->k_splits >= 2 && p->k_splits <= 8) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 1; attr[1].val.clusterDim.y = p->k_splits; attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
        static int ok_cache[2][9] = {{0}};                      // 0 unknown, 1 fits, -1 does not
        int& ok = ok_cache[fast][p->k_splits];
        if (ok == 0) {
            int n = 0;
            cudaError_t e = fast ? cudaOccupancyMaxActiveClusters(&n, gemv_int4_kernel<true>, &cfg)
                                 : cudaOccupancyMaxActiveClusters(&n, gemv_int4_kernel<false>, &cfg);
            ok = (e == cudaSuccess && n >= 1) ? 1 : -1;
            if (e != cudaSuccess) cudaGetLastError();
        }
        if (ok == 1) q.cluster_splitk = 1; else cfg.numAttrs = 1;
    }
    if (fast) return cudaLaunchKernelEx(&cfg, gemv_int4_kernel<true>, q);
    return cudaLaunchKernelEx(&cfg, gemv_int4_kernel<false>, q);
}

template <int MR>
static int launch_f16(const GemvF16Params* p, cudaStream_t stream) {
    size_t smem = (size_t)MR * p->kslice * 2 + (B2_MAX_ROWS * GEMV_TILE_N + 32 + 4) * 4;
    static SmemOptIn optin;
    {
        cudaError_t e = optin.ensure(gemv_f16_kernel<MR>, smem);
        if (e != cudaSuccess) return e;
    }
    dim3 grid((p->N + GEMV_TILE_N - 1) / GEMV_TILE_N, p->k_splits);
    // A plain launch: with the programmatic-serialisation attribute this kernel (nothing to do before its
    // dependency wait, 40-170 MB to stream after it) measured 10 % slower in the decode step (fp16 attention
    // weights: 149.1 against 167.1 tok/s).
    gemv_f16_kernel<MR><<<grid, GEMV_THREADS, smem, stream>>>(*p);
    return cudaGetLastError();
}

B2_API int b2_gemv_f16(const GemvF16Params* p, cudaStream_t stream) {
    if (p->rows < 1 || p->rows > B2_MAX_ROWS || (p->kslice & 255)) return cudaErrorInvalidValue;
    if (p->epi.mode == EPI_FINISH && p->epi.n_valid > 8192) return cudaErrorInvalidValue;
    if (p->rows == 1) return launch_f16<1>(p, stream);
    if (p->rows == 2) return launch_f16<2>(p, stream);
    if (p->rows <= 4) return launch_f16<4>(p, stream);
    return launch_f16<8>(p, stream);
}

B2_API int b2_sizeof_gemv_int4_params() { return (int)sizeof(GemvInt4Params); }
B2_API int b2_sizeof_gemv_f16_params() { return (int)sizeof(GemvF16Params); }
B2_API int b2_sizeof_comm_ctx() { return (int)sizeof(CommCtx); }

// ---------------------------------------------------------------------------
// Allocation-free entry point (see gemv_noalloc.h).  The scratch block is a file-scope
// device array; in host code its name is only a handle, so the device address is looked
// up once per device with cudaGetSymbolAddress and that pointer is what the kernel gets.
// ---------------------------------------------------------------------------
#include <mutex>
#include "gemv_noalloc.h"

#define B2_NOALLOC_COUNTER_BYTES 4096u
#define B2_NOALLOC_MAX_DEVICES 64

static __device__ __align__(256) unsigned char b2_noalloc_scratch[B2_NOALLOC_SCRATCH_BYTES];

static void noalloc_launch_shape(int KB, int NTL, int rows, int* k_splits, int* L) {
    // same choice as ops/packing.py:launch_shape: fill 2 x 148 CTA slots in one wave, even L
    const int ctas_n = NTL * 16 / GEMV_TILE_N;
    int ks = (2 * 148) / (ctas_n > 0 ? ctas_n : 1);
    const int ks_max = (KB + GEMV_WK - 1) / GEMV_WK;
    if (ks > ks_max) ks = ks_max;
    if (ks < 1) ks = 1;
    if (KB <= 24) ks = 1;                          // short K: no cross-CTA split (as ops/packing.py)
    auto even = [&](int v) { return (KB >= 2 * GEMV_WK) ? v + (v & 1) : v; };
    int l = even((KB + GEMV_WK * ks - 1) / (GEMV_WK * ks));
    while ((size_t)2 * GEMV_WK * l * (rows + 1) * 64 > 32000u) {
        ++ks;
        l = even((KB + GEMV_WK * ks - 1) / (GEMV_WK * ks));
    }
    *L = l;
    *k_splits = (KB + GEMV_WK * l - 1) / (GEMV_WK * l);
}

B2_API size_t b2_gemv_int4_noalloc_required(int rows, int K, int N) {
    if (rows < 1 || K < 8 || N < 1) return 0;
    const int KB = (K + 63) / 64, NTL = (N + GEMV_TILE_N - 1) / GEMV_TILE_N * (GEMV_TILE_N / 16);
    int ks, L;
    noalloc_launch_shape(KB, NTL, rows, &ks, &L);
    const size_t partial = ks > 1 ? (size_t)ks * rows * NTL * 16 * sizeof(float) : 0;
    return B2_NOALLOC_COUNTER_BYTES + partial;
}

B2_API const char* b2_gemv_int4_noalloc_strerror(int code) {
    switch (code) {
        case B2_NOALLOC_OK: return "ok";
        case B2_NOALLOC_ERR_BAD_ARGUMENT:
            return "bad argument: null pointer, rows outside 1..8, K not a multiple of 8, unsupported group size/offset, "
                   "odd ldx, or a misaligned pointer (x: 4 bytes, out: 2, qfrag: 16, szfrag: 8)";
        case B2_NOALLOC_ERR_TOO_LARGE:
            return "problem needs more scratch than the built-in block (B2_NOALLOC_SCRATCH_BYTES); use b2_gemv_int4 with a caller-provided buffer";
        case B2_NOALLOC_ERR_SYMBOL: return "could not obtain the device address of the built-in scratch block";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
    }
}

B2_API int b2_gemv_int4_noalloc(const void* qfrag, const void* szfrag, const void* x, int ldx, void* out, int ldo,
                                int rows, int K, int N, int group_size, int group_offset, cudaStream_t stream) {
    if (!qfrag || !szfrag || !x || !out || rows < 1 || rows > B2_MAX_ROWS || K < 8 || (K & 7) || N < 1 ||
        ldx < K || ldo < N)
        return B2_NOALLOC_ERR_BAD_ARGUMENT;
    // the kernel reads activations as fp16 pairs, weights as 16-byte words and scale/zero entries as
    // 8-byte words: a pointer or stride that breaks those alignments would fault on the device
    if ((ldx & 1) || ((uintptr_t)x & 3) || ((uintptr_t)out & 1) || ((uintptr_t)qfrag & 15) || ((uintptr_t)szfrag & 7))
        return B2_NOALLOC_ERR_BAD_ARGUMENT;
    int gshift;
    switch (group_size) {
        case 32: gshift = 0; break;
        case 64: gshift = 1; break;
        case 128: gshift = 2; break;
        case 256: gshift = 3; break;
        default: return B2_NOALLOC_ERR_BAD_ARGUMENT;
    }
    if (group_offset < 0 || group_offset >= group_size || (group_offset & 31)) return B2_NOALLOC_ERR_BAD_ARGUMENT;
    const int KB = (K + 63) / 64, NTL = (N + GEMV_TILE_N - 1) / GEMV_TILE_N * (GEMV_TILE_N / 16);
    if ((size_t)(NTL * 16 / GEMV_TILE_N + 1) * sizeof(int) > B2_NOALLOC_COUNTER_BYTES) return B2_NOALLOC_ERR_TOO_LARGE;
    if (b2_gemv_int4_noalloc_required(rows, K, N) > B2_NOALLOC_SCRATCH_BYTES) return B2_NOALLOC_ERR_TOO_LARGE;

    // ---- once per device: device address of the scratch block (the current device's copy)
    static std::mutex mu;
    static unsigned char* dev_ptr[B2_NOALLOC_MAX_DEVICES] = {nullptr};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= B2_NOALLOC_MAX_DEVICES) return B2_NOALLOC_ERR_SYMBOL;
    unsigned char* base;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!dev_ptr[dev]) {
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, b2_noalloc_scratch);
            if (e != cudaSuccess || !ptr) return B2_NOALLOC_ERR_SYMBOL;
            dev_ptr[dev] = (unsigned char*)ptr;
        }
        base = dev_ptr[dev];
    }
    // ---- counters must start at zero; partial sums are overwritten before they are read
    e = cudaMemsetAsync(base, 0, B2_NOALLOC_COUNTER_BYTES, stream);
    if (e != cudaSuccess) return (int)e;

    GemvInt4Params p;
    memset(&p, 0, sizeof(p));
    p.qfrag = (const uint4*)qfrag; p.szfrag = (const uint2*)szfrag; p.x = (const __half*)x;
    p.ldx = ldx; p.rows = rows; p.K = K; p.KB = KB; p.NTL = NTL;
    p.G = (KB * 64 + group_offset + group_size - 1) / group_size;
    p.off32 = group_offset / 32; p.gshift = gshift;
    noalloc_launch_shape(KB, NTL, rows, &p.k_splits, &p.L);
    p.counters = (int*)base;
    p.scratch = (float*)(base + B2_NOALLOC_COUNTER_BYTES);
    p.epi.mode = EPI_STORE_F16; p.epi.out = out; p.epi.ldo = ldo; p.epi.n_valid = N;
    p.comm.tp = 1;
    return b2_gemv_int4(&p, stream);
}
