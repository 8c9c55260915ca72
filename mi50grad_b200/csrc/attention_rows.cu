// Tensor-core attention over the KV cache for many query rows: prompt processing, draft
// verification and batched decode.
//
// Rows of one sequence are taken 16 at a time; a CTA handles one such tile for one KV head and
// (optionally) one slice of the cache, with one warp per query head of the GQA group, so K and V
// are staged in shared memory once per group.  S = Q K^T and O += P V run on mma.sync m16n8k16
// (fp16 in, fp32 accumulate) with the online-softmax rescaling of flash attention; the visibility
// rule is the decode kernel's:  slot s is visible to a row iff  s < ctx  or  bit (s - ctx) of its
// mask is set, which covers causal prompts (ctx = position + 1) and draft trees (ctx = committed
// length, mask = the node's ancestors and itself).  The sigmoid output gate is applied in the
// epilogue.  This replaces the reference's prefill attention kernels and its tree-masked variant
// (reference: src/kernels/flash_attn_256.hip, src/kernels/flash_attn_256_v3.hip,
// src/kernels/flash_attn_tree.hip:74-193), which walk the keys with scalar dot products.
#include "kernels.cuh"

#define AR_ROWS 16               // query rows per tile
#define AR_KV 64                 // cache slots per block
#define AR_MAX_WARPS 8
#define AR_PAD 8                 // halfs of padding per shared-memory row (conflict-free ldmatrix)

__device__ __forceinline__ void ar_ldsm4(uint32_t (&r)[4], const __half* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ar_ldsm4_t(uint32_t (&r)[4], const __half* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ar_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float x, float y) {
    __half2 h = __floats2half2_rn(x, y);
    return *(uint32_t*)&h;
}

// Find the tile: sequences are consecutive row ranges (seq_rows), each cut into 16-row tiles.
__device__ __forceinline__ bool ar_find_tile(const int* seq_rows, int n_seqs, int tile, int& row0, int& nrows) {
    for (int s = 0; s < n_seqs; ++s) {
        const int a = seq_rows[s], b = seq_rows[s + 1];
        const int nt = (b - a + AR_ROWS - 1) / AR_ROWS;
        if (tile < nt) { row0 = a + tile * AR_ROWS; nrows = min(AR_ROWS, b - row0); return true; }
        tile -= nt;
    }
    return false;
}

template <int HD>
__global__ void __launch_bounds__(AR_MAX_WARPS * 32, 1) attn_rows_kernel(const AttnParams p, const int* __restrict__ seq_rows,
                                                                        int n_seqs, int splits) {
    constexpr int LD = HD + AR_PAD;
    constexpr int NT_O = HD / 8;                 // 8-column tiles of the output
    pdl_launch_dependents();
    int row0, nrows;
    if (!ar_find_tile(seq_rows, n_seqs, blockIdx.x, row0, nrows)) return;
    const int kvh = blockIdx.y, sp = blockIdx.z;
    const int G = p.nq / p.nkv;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthr = blockDim.x;
    const int g = lane >> 2, t = lane & 3;

    extern __shared__ __align__(16) unsigned char ar_smem[];
    __half* Qs = (__half*)ar_smem;                               // [G][16][LD]
    __half* Kb = Qs + (size_t)G * AR_ROWS * LD;                  // [2][64][LD]
    __half* Vb = Kb + 2 * AR_KV * LD;                            // [2][64][LD]

    // visibility of this thread's two rows (g and g + 8 of the tile)
    const RowMeta r_lo = p.rows[row0 + min(g, nrows - 1)], r_hi = p.rows[row0 + min(g + 8, nrows - 1)];
    const int ctx_lo = g < nrows ? r_lo.ctx : 0, ctx_hi = g + 8 < nrows ? r_hi.ctx : 0;
    const unsigned long long mk_lo = g < nrows ? r_lo.mask : 0ull, mk_hi = g + 8 < nrows ? r_hi.mask : 0ull;
    const int seq = r_lo.seq;
    // cache range the tile needs: the furthest visible slot over its rows (every thread computes the same value)
    int kv_end = 0;
    for (int r = 0; r < nrows; ++r) {
        const RowMeta rm = p.rows[row0 + r];
        const int extra = rm.mask ? 64 - __clzll((long long)rm.mask) : 0;
        kv_end = max(kv_end, min(rm.ctx + extra, p.max_seq));
    }
    const int n_blocks = (kv_end + AR_KV - 1) / AR_KV;
    const int per = (n_blocks + splits - 1) / splits;
    const int b_begin = sp * per, b_end = min(n_blocks, b_begin + per);

    // ---- stage Q (all heads of the group) and the first K/V block
    const size_t kv_base = ((size_t)seq * p.max_seq) * p.nkv * HD + (size_t)kvh * HD;
    const size_t kv_stride = (size_t)p.nkv * HD;
    constexpr int PPR = HD / 8;                                  // 16-byte pieces per row
    for (int idx = tid; idx < G * AR_ROWS * PPR; idx += nthr) {
        const int pc = idx % PPR, r = (idx / PPR) % AR_ROWS, h = idx / (PPR * AR_ROWS);
        __half* dst = Qs + ((size_t)h * AR_ROWS + r) * LD + pc * 8;
        if (r < nrows) cp_async16(dst, p.q + (size_t)(row0 + r) * p.ldq + (size_t)(kvh * G + h) * HD + pc * 8);
        else *(uint4*)dst = make_uint4(0u, 0u, 0u, 0u);
    }
    auto stage_kv = [&](int blk, int buf) {
        for (int idx = tid; idx < AR_KV * PPR; idx += nthr) {
            const int pc = idx % PPR, r = idx / PPR;
            const int slot = blk * AR_KV + r;
            __half* kd = Kb + ((size_t)buf * AR_KV + r) * LD + pc * 8;
            __half* vd = Vb + ((size_t)buf * AR_KV + r) * LD + pc * 8;
            if (slot < kv_end) {
                cp_async16(kd, p.kcache + kv_base + (size_t)slot * kv_stride + pc * 8);
                cp_async16(vd, p.vcache + kv_base + (size_t)slot * kv_stride + pc * 8);
            } else {
                *(uint4*)kd = make_uint4(0u, 0u, 0u, 0u);
                *(uint4*)vd = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
    if (b_begin < b_end) stage_kv(b_begin, 0);
    cp_async_commit();

    float o[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    const bool active = warp < G;
    const __half* qw = Qs + (size_t)warp * AR_ROWS * LD;
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;      // A operand (row-major) addressing
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;      // B operand from [n][k] storage
    const float sc = p.scale * 1.44269504f;                      // scores are kept in the log2 domain

    for (int blk = b_begin; blk < b_end; ++blk) {
        const int buf = (blk - b_begin) & 1;
        cp_async_wait<0>();
        __syncthreads();                                         // block `blk` landed; everyone left block blk-1
        if (blk + 1 < b_end) stage_kv(blk + 1, buf ^ 1);
        cp_async_commit();
        if (!active) continue;
        const __half* Kt = Kb + (size_t)buf * AR_KV * LD;
        const __half* Vt = Vb + (size_t)buf * AR_KV * LD;
        // ---- S = Q K^T  (16 x 64)
        float s[AR_KV / 8][4];
#pragma unroll
        for (int n = 0; n < AR_KV / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll 2
        for (int k0 = 0; k0 < HD; k0 += 16) {
            uint32_t a[4];
            ar_ldsm4(a, qw + a_row * LD + k0 + a_col);
#pragma unroll
            for (int np = 0; np < AR_KV / 16; ++np) {
                uint32_t b[4];
                ar_ldsm4(b, Kt + (np * 16 + b_row) * LD + k0 + b_col);
                ar_mma(s[2 * np], a, b[0], b[1]);
                ar_mma(s[2 * np + 1], a, b[2], b[3]);
            }
        }
        // ---- mask, online softmax
        const int s_base = blk * AR_KV;
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int n = 0; n < AR_KV / 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int slot = s_base + 8 * n + 2 * t + (e & 1);
                const bool hi = e >= 2;
                const int ctx = hi ? ctx_hi : ctx_lo;
                const unsigned long long mk = hi ? mk_hi : mk_lo;
                const int d = slot - ctx;
                const bool vis = d < 0 || (d < 64 && ((mk >> d) & 1ull));
                const float v = vis ? s[n][e] * sc : -INFINITY;
                s[n][e] = v;
                if (hi) mx_hi = fmaxf(mx_hi, v); else mx_lo = fmaxf(mx_lo, v);
            }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float ref_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float cor_lo = exp2f(m_lo - ref_lo), cor_hi = exp2f(m_hi - ref_hi);      // exp2(-inf) = 0 for the first block
        m_lo = mn_lo; m_hi = mn_hi;
        float rs_lo = 0.f, rs_hi = 0.f;
        uint32_t pa[AR_KV / 16][4];
#pragma unroll
        for (int n = 0; n < AR_KV / 8; ++n) {
            const float p0 = exp2f(s[n][0] - ref_lo), p1 = exp2f(s[n][1] - ref_lo);
            const float p2 = exp2f(s[n][2] - ref_hi), p3 = exp2f(s[n][3] - ref_hi);
            rs_lo += p0 + p1; rs_hi += p2 + p3;
            // two adjacent 8-column score tiles form the A fragment of one 16-slot step of P V
            pa[n >> 1][(n & 1) * 2 + 0] = pack_h2(p0, p1);
            pa[n >> 1][(n & 1) * 2 + 1] = pack_h2(p2, p3);
        }
        l_lo = l_lo * cor_lo + rs_lo; l_hi = l_hi * cor_hi + rs_hi;
#pragma unroll
        for (int n = 0; n < NT_O; ++n) { o[n][0] *= cor_lo; o[n][1] *= cor_lo; o[n][2] *= cor_hi; o[n][3] *= cor_hi; }
        // ---- O += P V
#pragma unroll
        for (int k16 = 0; k16 < AR_KV / 16; ++k16) {
#pragma unroll
            for (int np = 0; np < NT_O / 2; ++np) {
                uint32_t b[4];
                ar_ldsm4_t(b, Vt + (k16 * 16 + a_row) * LD + np * 16 + a_col);
                ar_mma(o[2 * np], pa[k16], b[0], b[1]);
                ar_mma(o[2 * np + 1], pa[k16], b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    if (!active) return;
    // row sums live in the four lanes of a row quad
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const int head = kvh * G + warp;
    if (splits == 1) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = g + 8 * half;
            if (r >= nrows) continue;
            const float inv = 1.f / (half ? l_hi : l_lo);
            const size_t row = (size_t)(row0 + r);
#pragma unroll
            for (int n = 0; n < NT_O; ++n) {
                const int col = 8 * n + 2 * t;
                float v0 = o[n][2 * half] * inv, v1 = o[n][2 * half + 1] * inv;
                if (p.gate_off >= 0) {
                    const __half2 gt = *(const __half2*)(p.q + row * p.ldq + p.gate_off + (size_t)head * HD + col);
                    v0 *= sigmoid_f(__low2float(gt)); v1 *= sigmoid_f(__high2float(gt));
                }
                *(__half2*)(p.out + row * p.ldo + (size_t)head * HD + col) = __floats2half2_rn(v0, v1);
            }
        }
    } else {
        // partial result of this slice: unnormalised O, running maximum (log2 domain) and sum
        // scratch: [row][head][split][HD + 2]
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = g + 8 * half;
            if (r >= nrows) continue;
            float* dst = p.scratch + (((size_t)(row0 + r) * p.nq + head) * splits + sp) * (HD + 2);
#pragma unroll
            for (int n = 0; n < NT_O; ++n)
                *(float2*)(dst + 8 * n + 2 * t) = make_float2(o[n][2 * half], o[n][2 * half + 1]);
            if (t == 0) { dst[HD] = half ? m_hi : m_lo; dst[HD + 1] = half ? l_hi : l_lo; }
        }
    }
}

// Merge the slices of split attention: one warp per (row, head).
template <int HD>
__global__ void __launch_bounds__(128) attn_rows_merge_kernel(const AttnParams p, int splits) {
    pdl_launch_dependents();
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= p.n_rows * p.nq) return;
    const int row = item / p.nq, head = item % p.nq;
    const float* src = p.scratch + (size_t)item * splits * (HD + 2);
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, src[(size_t)s * (HD + 2) + HD]);
    if (m == -INFINITY) m = 0.f;
    constexpr int EPL = HD / 32;
    float acc[EPL], l = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float* ps = src + (size_t)s * (HD + 2);
        const float w = exp2f(ps[HD] - m);
        l += ps[HD + 1] * w;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] += ps[lane * EPL + e] * w;
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        const int col = lane * EPL + e;
        float v = acc[e] * inv;
        if (p.gate_off >= 0) v *= sigmoid_f(__half2float(p.q[(size_t)row * p.ldq + p.gate_off + (size_t)head * HD + col]));
        p.out[(size_t)row * p.ldo + (size_t)head * HD + col] = __float2half(v);
    }
}

template <int HD>
static int launch_rows(const AttnParams* p, const int* seq_rows, int n_seqs, int splits, cudaStream_t s) {
    const int G = p->nq / p->nkv;
    const size_t smem = ((size_t)G * AR_ROWS + 4 * AR_KV) * (HD + AR_PAD) * sizeof(__half);
    static SmemOptIn optin;
    {
        cudaError_t e = optin.ensure(attn_rows_kernel<HD>, smem);
        if (e != cudaSuccess) return e;
    }
    const int tiles = (p->n_rows + AR_ROWS - 1) / AR_ROWS + n_seqs;       // upper bound; surplus CTAs exit at once
    dim3 grid(tiles, p->nkv, splits);
    attn_rows_kernel<HD><<<grid, G * 32, smem, s>>>(*p, seq_rows, n_seqs, splits);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || splits == 1) return e;
    attn_rows_merge_kernel<HD><<<(p->n_rows * p->nq + 3) / 4, 128, 0, s>>>(*p, splits);
    return cudaGetLastError();
}

// p->splits: cache slices per tile (1 = none; needs scratch of n_rows * nq * splits * (hd + 2) floats).
B2_API int b2_attn_rows(const AttnParams* p, const int* seq_rows, int n_seqs, int hd, cudaStream_t s) {
    const int G = p->nkv > 0 ? p->nq / p->nkv : 0;
    if (G < 1 || G > AR_MAX_WARPS || p->nq % p->nkv || n_seqs < 1 || p->splits < 1) return cudaErrorInvalidValue;
    if (hd == 256) return launch_rows<256>(p, seq_rows, n_seqs, p->splits, s);
    if (hd == 64) return launch_rows<64>(p, seq_rows, n_seqs, p->splits, s);
    return cudaErrorInvalidValue;
}
