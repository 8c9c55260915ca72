// Causal prompt attention on the 5th-generation tensor cores (tcgen05 + tensor memory + TMA).
//
// One CTA owns 128 consecutive query rows of one query head of one sequence and walks the KV cache in
// tiles of 64 slots up to the last slot its rows may see:
//   S = Q K^T        tcgen05.mma, M = 128 rows, N = 64 slots, K = head dim; Q and the K tile arrive by TMA
//                    (128-byte swizzle, no cluster broadcast) in the K-major layout the MMA reads;
//   soft-max         every thread owns one row of S in tensor memory (tcgen05.ld): masking, running
//                    max / sum and the fp16 probabilities need no shuffles; P goes to shared memory
//                    in the same swizzled K-major layout (it is the A operand of the second product);
//   O_tile = P V     tcgen05.mma, M = 128 rows, N = head dim, K = 64 slots; V is stored in the cache
//                    with the head dim contiguous, the MMA wants the slots contiguous, so the threads
//                    transpose the V tile (staged by cp.async) into shared memory while S is computed;
//   the K tile (TMA, two buffers) and the raw V tile (cp.async) of the next step are requested one step
//   ahead, so no step waits on global memory;
//   O = O * corr + O_tile in registers (each of the two warps of a tensor-memory lane quarter keeps half
//   of the head dim), then 1 / sum, the sigmoid output gate and the fp16 store.
// Grouped-query heads share the K/V tiles through L2.  Every mbarrier wait is bounded; on expiry the
// kernel records a status, frees its tensor memory and returns.
//
// Replaces the reference's prefill attention kernels, which run 64-wide tiles on vector ALUs
// (reference: src/kernels/flash_attn_256_v3.hip:80,189, flash_attn_256_tuned.hip:200).
#include <cuda.h>
#include "kernels.cuh"
#include "tc_util.cuh"

#define AT_ROWS 128               // query rows per CTA (MMA M)
#define AT_KV 64                  // cache slots per tile
#define AT_THREADS 256

// byte offset of (row, 16-byte chunk c8 of its 128-byte line) in a K-major 128-byte-swizzled tile
__device__ __forceinline__ uint32_t at_sw(int row, int c8) { return (uint32_t)row * 128u + (uint32_t)((c8 ^ (row & 7)) << 4); }

__device__ __forceinline__ void tc_ld32f(uint32_t taddr, float (&f)[32]) {
    uint32_t r[32];
    tc_ld32(taddr, r);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
}

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_prefill_tc_kernel(const AttnParams p, const __grid_constant__ CUtensorMap qmap,
                       const __grid_constant__ CUtensorMap kmap, int row_base, int n_rows_seq, int* status) {
    constexpr int NB = HD / 64;                   // 64-wide blocks of the head dim (one swizzle line each)
    constexpr int OC = HD / 2;                    // output columns per thread
    extern __shared__ __align__(1024) unsigned char at_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)at_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = smem;                                 // [NB][128 rows][128 B]
    constexpr int KB_BYTES = NB * AT_KV * 128;                // one K tile
    constexpr int VR_LD = HD * 2 + 16;                        // bytes per raw V row (padded: conflict-free transposition)
    unsigned char* sK = sQ + (size_t)NB * AT_ROWS * 128;      // [2][NB][64 slots][128 B]
    unsigned char* sVt = sK + (size_t)2 * KB_BYTES;           // [HD rows][128 B]: V transposed (slots contiguous)
    unsigned char* sP = sVt + (size_t)HD * 128;               // [128 rows][128 B]
    unsigned char* sVr = sP + (size_t)AT_ROWS * 128;          // [64 slots][VR_LD]: raw V tile of the next step
    uint64_t* bars = (uint64_t*)(sVr + (size_t)AT_KV * VR_LD); // [0], [3] K tiles (+ Q), [1] S ready, [2] O tile ready
    uint32_t* tmem_slot = (uint32_t*)(bars + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.y, kvh = head / (p.nq / p.nkv);
    const int r0 = row_base + blockIdx.x * AT_ROWS;           // first row of this CTA in the launch
    const int r_end = row_base + n_rows_seq;
    constexpr int tmem_cols = HD == 256 ? 512 : (HD == 128 ? 256 : 128);

    if (tid == 0) {
        mbar_init(&bars[0], 1); mbar_init(&bars[1], 1); mbar_init(&bars[2], 1); mbar_init(&bars[3], 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + AT_KV;

    // this thread's row: lane quarter (warp & 3) of tensor memory, row = 32 * (warp & 3) + lane
    const int lq = warp & 3, half = warp >> 2;
    const int row = lq * 32 + lane;
    const int gr = r0 + row;                                   // row in the launch
    const bool row_ok = gr < r_end;
    const RowMeta rm0 = p.rows[r0];
    const int seq = rm0.seq;
    const int my_ctx = row_ok ? p.rows[gr].ctx : 0;
    const int last = min(r0 + AT_ROWS, r_end) - 1;
    const int max_ctx = p.rows[last].ctx;                      // rows are in position order: the last sees the most
    const int n_tiles = (max_ctx + AT_KV - 1) / AT_KV;

    float o_acc[OC];
#pragma unroll
    for (int i = 0; i < OC; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const uint32_t idesc_s = make_idesc_f16(AT_KV), idesc_o = make_idesc_f16(HD);
    const uint64_t dQ = make_desc_sw128(smem_u32(sQ)), dK = make_desc_sw128(smem_u32(sK));
    const uint64_t dP = make_desc_sw128(smem_u32(sP)), dV = make_desc_sw128(smem_u32(sVt));
    const size_t vstride = (size_t)p.nkv * HD;
    const __half* vbase = p.vcache + ((size_t)seq * p.max_seq) * vstride + (size_t)kvh * HD;
    bool ok = true;

    // K tile t goes to buffer t & 1 on barrier (t & 1 ? 3 : 0); the raw V tile t to sVr
    auto issue_k = [&](int t) {
        if (warp == 0 && elect_one()) {
            uint64_t* bar = &bars[(t & 1) ? 3 : 0];
            const uint32_t bytes = (uint32_t)KB_BYTES + (t == 0 ? (uint32_t)NB * AT_ROWS * 128 : 0u);
            mbar_arrive_expect_tx(bar, bytes);
            if (t == 0)
                for (int b = 0; b < NB; ++b) tma_load_2d(sQ + (size_t)b * AT_ROWS * 128, &qmap, head * HD + b * 64, r0, bar);
            for (int b = 0; b < NB; ++b)
                tma_load_2d(sK + (size_t)(t & 1) * KB_BYTES + (size_t)b * AT_KV * 128, &kmap, kvh * HD + b * 64,
                            seq * p.max_seq + t * AT_KV, bar);
        }
    };
    auto issue_v = [&](int t) {
#pragma unroll
        for (int it = 0; it < HD / 32; ++it) {
            const int idx = tid + AT_THREADS * it, slot = idx / (HD / 8), ch = idx % (HD / 8);
            if (t * AT_KV + slot < max_ctx)
                cp_async16(sVr + (size_t)slot * VR_LD + ch * 16, vbase + (size_t)(t * AT_KV + slot) * vstride + ch * 8);
        }
        cp_async_commit();
    };
    if (n_tiles > 0) { issue_k(0); issue_v(0); }

    for (int tile = 0; tile < n_tiles && ok; ++tile) {
        const int kv0 = tile * AT_KV;
        const uint32_t par = (uint32_t)(tile & 1);
        if (tile + 1 < n_tiles) issue_k(tile + 1);             // its buffer was last read by the S product of tile - 1
        // ---- S = Q K^T (the K tile was requested a step ago)
        if (warp == 0) {
            const bool ok0 = mbar_wait(&bars[(tile & 1) ? 3 : 0], (uint32_t)((tile >> 1) & 1), abort_flag);
            tc_fence_after();
            if (ok0 && elect_one()) {
                const uint64_t dKt = dK + (uint64_t)(((tile & 1) * KB_BYTES) >> 4);
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16)
                        tc_mma_f16(tmem_S, dQ + (uint64_t)((b * AT_ROWS * 128) >> 4) + 2 * k16,
                                   dKt + (uint64_t)((b * AT_KV * 128) >> 4) + 2 * k16, idesc_s, (b | k16) ? 1u : 0u);
                tc_commit(&bars[1]);
            }
            __syncwarp();
        }
        // ---- meanwhile: transpose the raw V tile into the layout the second product reads
        cp_async_wait<0>();
        __syncthreads();
        {
            const int j = tid & 63;                             // slot of the tile
            const bool live = kv0 + j < max_ctx;
#pragma unroll
            for (int it = 0; it < HD / 32; ++it) {
                const int d0 = ((tid >> 6) + 4 * it) * 8;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (live) v = *(const uint4*)(sVr + (size_t)j * VR_LD + d0 * 2);
                const __half* hv = (const __half*)&v;
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    *(__half*)(sVt + at_sw(d0 + e, j >> 3) + (j & 7) * 2) = hv[e];
            }
        }
        fence_proxy_async_smem();
        __syncthreads();
        if (tile + 1 < n_tiles) issue_v(tile + 1);              // flies while this tile is processed
        // (a thread whose wait gave up still walks to the next barrier, where the whole CTA decides to stop)
        const bool ok1 = mbar_wait(&bars[1], par, abort_flag);
        tc_fence_after();
        // ---- soft-max over this tile's 64 scores of the row (pass 1: max, pass 2: probabilities)
        float s[32];
        float m_new = m_run;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            tc_ld32f(tmem_S + ((uint32_t)(lq * 32) << 16) + c * 32, s);
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (kv0 + c * 32 + i < my_ctx) m_new = fmaxf(m_new, s[i] * p.scale);
        }
        const float corr = (m_new == -INFINITY) ? 1.f : __expf(m_run - m_new);
        float psum = 0.f;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            tc_ld32f(tmem_S + ((uint32_t)(lq * 32) << 16) + c * 32, s);
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float p0 = (kv0 + c * 32 + i < my_ctx) ? __expf(s[i] * p.scale - m_new) : 0.f;
                const float p1 = (kv0 + c * 32 + i + 1 < my_ctx) ? __expf(s[i + 1] * p.scale - m_new) : 0.f;
                const __half2 h2 = __floats2half2_rn(p0, p1);
                // the sum uses the rounded values the second product sees
                psum += __low2float(h2) + __high2float(h2);
                pk[i >> 1] = *(const uint32_t*)&h2;
            }
            if (half == c) {                                   // the two warps of a lane quarter write half a row each
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    *(uint4*)(sP + at_sw(row, c * 4 + q)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
            }
        }
        l_run = l_run * corr + psum;
        m_run = m_new;
        fence_proxy_async_smem();
        tc_fence_before();
        ok = __syncthreads_and(ok1 ? 1 : 0) != 0;
        if (!ok) break;
        // ---- O_tile = P V
        if (warp == 0) {
            tc_fence_after();
            if (elect_one()) {
#pragma unroll
                for (int k16 = 0; k16 < AT_KV / 16; ++k16)
                    tc_mma_f16(tmem_O, dP + 2 * k16, dV + 2 * k16, idesc_o, k16 ? 1u : 0u);
                tc_commit(&bars[2]);
            }
            __syncwarp();
        }
        const bool ok2 = mbar_wait(&bars[2], par, abort_flag);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < OC / 32; ++c) {
            tc_ld32f(tmem_O + ((uint32_t)(lq * 32) << 16) + half * OC + c * 32, s);
#pragma unroll
            for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * corr + s[i];
        }
        tc_fence_before();
        ok = __syncthreads_and(ok2 ? 1 : 0) != 0;              // shared memory and tensor memory are free again
    }

    if (ok && row_ok) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        const size_t col0 = (size_t)head * HD + half * OC;
        __half* dst = p.out + (size_t)gr * p.ldo + col0;
        const __half* gq = p.gate_off >= 0 ? p.q + (size_t)gr * p.ldq + p.gate_off + col0 : nullptr;
#pragma unroll
        for (int c = 0; c < OC; c += 8) {
            uint4 gv = make_uint4(0u, 0u, 0u, 0u);
            if (gq) gv = *(const uint4*)(gq + c);
            const __half* gh = (const __half*)&gv;
            __half2 o2[4];
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
                float a = o_acc[c + e] * inv, b = o_acc[c + e + 1] * inv;
                if (gq) { a *= sigmoid_f(__half2float(gh[e])); b *= sigmoid_f(__half2float(gh[e + 1])); }
                o2[e >> 1] = __floats2half2_rn(a, b);
            }
            *(uint4*)(dst + c) = *(const uint4*)o2;
        }
    }
    if (*abort_flag && tid == 0 && status) atomicExch(status, 1);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(tmem_cols) : "memory");
}

static size_t at_smem(int hd) {
    const int nb = hd / 64;
    return 1024 + (size_t)nb * AT_ROWS * 128 + (size_t)2 * nb * AT_KV * 128 + (size_t)hd * 128 + (size_t)AT_ROWS * 128 +
           (size_t)AT_KV * (hd * 2 + 16) + 64;
}

template <int HD>
static int launch_attn_prefill_tc(const AttnParams* p, const CUtensorMap& qmap, const CUtensorMap& kmap, int row_base,
                                  int n_rows_seq, int* status, cudaStream_t s) {
    const size_t smem = at_smem(HD);
    static SmemOptIn opt;
    if (int e = opt.ensure(attn_prefill_tc_kernel<HD>, smem)) return e;
    dim3 grid((n_rows_seq + AT_ROWS - 1) / AT_ROWS, p->nq);
    attn_prefill_tc_kernel<HD><<<grid, AT_THREADS, smem, s>>>(*p, qmap, kmap, row_base, n_rows_seq, status);
    return cudaGetLastError();
}

// Rows [row_base, row_base + n_rows_seq) of the launch belong to one sequence, are in position order and carry
// no draft-tree masks (RowMeta.mask == 0); the cache already holds their own K/V rows.  n_slots: sequence slots
// of the cache (its first dimension).  status[0] is set to 1 when a bounded wait expired.
B2_API int b2_attn_prefill_tc(const AttnParams* p, int row_base, int n_rows_seq, int n_slots, int hd, int* status,
                              cudaStream_t s) {
    if (hd != 64 && hd != 128 && hd != 256) return cudaErrorInvalidValue;
    if (p->nq % p->nkv || n_rows_seq < 1 || (p->ldq & 7) || (p->ldo & 7) || ((uintptr_t)p->q & 15) || ((uintptr_t)p->out & 15) ||
        ((uintptr_t)p->kcache & 15) || ((uintptr_t)p->vcache & 15) || (p->gate_off >= 0 && (p->gate_off & 7)))
        return cudaErrorInvalidValue;
    EncodeTiledFn enc = get_encode();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap qmap, kmap;
    cuuint32_t estr[2] = {1, 1};
    {
        cuuint64_t dims[2] = {(cuuint64_t)p->nq * hd, (cuuint64_t)p->n_rows};
        cuuint64_t strides[1] = {(cuuint64_t)p->ldq * 2};
        cuuint32_t box[2] = {64, AT_ROWS};
        if (enc(&qmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)p->q, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)p->nkv * hd, (cuuint64_t)p->max_seq * n_slots};
        cuuint64_t strides[1] = {(cuuint64_t)p->nkv * hd * 2};
        cuuint32_t box[2] = {64, AT_KV};
        if (enc(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)p->kcache, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    if (hd == 256) return launch_attn_prefill_tc<256>(p, qmap, kmap, row_base, n_rows_seq, status, s);
    if (hd == 128) return launch_attn_prefill_tc<128>(p, qmap, kmap, row_base, n_rows_seq, status, s);
    return launch_attn_prefill_tc<64>(p, qmap, kmap, row_base, n_rows_seq, status, s);
}
