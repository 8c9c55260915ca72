// Decode / verify attention with a KV cache: split-KV flash decoding with an
// in-kernel merge, a sigmoid output gate and optional draft-tree masks.
//
// One kernel covers the reference's decode attention, its sigmoid gate and its
// tree-masked variant (reference: src/kernels/flash_attn_256_tuned.hip:171-350,
// src/kernels/sigmoid_mul.hip:10, src/kernels/flash_attn_tree.hip:74-193), with
// per-row sequence ids, lengths and masks read from device memory (RowMeta)
// instead of host-patched arguments.  Visibility of cache slot s for a row:
//     s < ctx   or   (s - ctx < 64 and mask bit (s - ctx) set).
//
// grid = (kv_heads, rows, splits); a CTA handles every query head of its KV
// head (GQA), so K/V are read once per group.  Each warp walks cache slots with
// stride, lanes split the head dimension (HD/32 elements each), scores are
// reduced with shuffles, and (max, sum, acc) are merged across warps in shared
// memory and across splits through a scratch buffer by the last CTA to arrive.
#include "kernels.cuh"

#define ATT_WARPS 4
#define ATT_THREADS (ATT_WARPS * 32)
#define ATT_MAX_G 8
#define ATT_MIN_SPLIT_LEN 32


template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) decode_attn_kernel(const AttnParams p) {
    constexpr int EPL = HD / 32;                 // elements per lane
    const int kvh = blockIdx.x, r = blockIdx.y, sp = blockIdx.z;
    pdl_launch_dependents();
    pdl_wait();                                  // Q, and the K/V row of this step, come from the kernels before
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = p.nq / p.nkv;
    const RowMeta rm = p.rows[r];
    const int extra = rm.mask ? 64 - __clzll((long long)rm.mask) : 0;
    const int total = rm.ctx + extra;
    // short contexts do not pay for a cross-CTA merge: one split per ATT_MIN_SPLIT_LEN slots
    const int nsplit = max(1, min(p.splits, (total + ATT_MIN_SPLIT_LEN - 1) / ATT_MIN_SPLIT_LEN));
    if (sp >= nsplit) return;
    const int per = (total + nsplit - 1) / nsplit;
    const int s0 = sp * per, s1 = min(total, s0 + per);

    __shared__ float sm_m[ATT_WARPS][ATT_MAX_G], sm_l[ATT_WARPS][ATT_MAX_G];
    __shared__ float sm_acc[ATT_WARPS][ATT_MAX_G][HD];
    __shared__ int s_last;
    __shared__ float sm_f[32][ATT_MAX_G], sm_linv[ATT_MAX_G];

    float q[ATT_MAX_G][EPL], acc[ATT_MAX_G][EPL], m[ATT_MAX_G], l[ATT_MAX_G];
#pragma unroll
    for (int h = 0; h < ATT_MAX_G; ++h) {
        m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            acc[h][e] = 0.f;
            q[h][e] = (h < G) ? __half2float(p.q[(size_t)r * p.ldq + (kvh * G + h) * HD + lane * EPL + e]) * p.scale : 0.f;
        }
    }
    const size_t base = ((size_t)rm.seq * p.max_seq) * p.nkv * HD + (size_t)kvh * HD + lane * EPL;
    const size_t stride = (size_t)p.nkv * HD;
    // K/V rows of the next slot are fetched while the current one is processed
    auto fetch = [&](int s, uint4& kv, uint4& vv) {
        const __half* kp = p.kcache + base + (size_t)s * stride;
        const __half* vp = p.vcache + base + (size_t)s * stride;
        if constexpr (EPL == 8) { kv = *(const uint4*)kp; vv = *(const uint4*)vp; }
        else if constexpr (EPL == 4) { kv.x = ((const uint2*)kp)->x; kv.y = ((const uint2*)kp)->y; vv.x = ((const uint2*)vp)->x; vv.y = ((const uint2*)vp)->y; }
        else { kv.x = *(const uint32_t*)kp; vv.x = *(const uint32_t*)vp; }
    };
    uint4 kv_n = make_uint4(0u, 0u, 0u, 0u), vv_n = kv_n;
    if (s0 + warp < s1) fetch(s0 + warp, kv_n, vv_n);
    for (int s = s0 + warp; s < s1; s += ATT_WARPS) {
        uint4 kv = kv_n, vv = vv_n;
        if (s + ATT_WARPS < s1) fetch(s + ATT_WARPS, kv_n, vv_n);
        bool vis = s < rm.ctx || ((rm.mask >> (s - rm.ctx)) & 1ull);
        if (!vis) continue;
        float kf[EPL], vf[EPL];
        {
            const __half2* k2 = (const __half2*)&kv; const __half2* v2 = (const __half2*)&vv;
#pragma unroll
            for (int e = 0; e < EPL / 2; ++e) {
                float2 a = __half22float2(k2[e]), b = __half22float2(v2[e]);
                kf[2 * e] = a.x; kf[2 * e + 1] = a.y; vf[2 * e] = b.x; vf[2 * e + 1] = b.y;
            }
        }
#pragma unroll
        for (int h = 0; h < ATT_MAX_G; ++h) {
            if (h < G) {
                float d = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) d = fmaf(q[h][e], kf[e], d);
                d = warp_sum(d);
                float mn = fmaxf(m[h], d);
                float corr = __expf(m[h] - mn), pw = __expf(d - mn);
                l[h] = l[h] * corr + pw;
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[h][e] = acc[h][e] * corr + pw * vf[e];
                m[h] = mn;
            }
        }
    }
    // ---- merge the warps of this CTA
#pragma unroll
    for (int h = 0; h < ATT_MAX_G; ++h) {
        if (h < G) {
            if (lane == 0) { sm_m[warp][h] = m[h]; sm_l[warp][h] = l[h]; }
#pragma unroll
            for (int e = 0; e < EPL; ++e) sm_acc[warp][h][lane * EPL + e] = acc[h][e];
        }
    }
    __syncthreads();
    // thread tid handles (h, d) pairs
    float* my = p.scratch + (((size_t)r * p.nkv + kvh) * p.splits + sp) * G * (HD + 2);
    const int splits_orig = p.splits;
    for (int i = tid; i < G * HD; i += ATT_THREADS) {
        int h = i / HD, d = i % HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, sm_m[w][h]);
        float ll = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) {
            float f = (sm_m[w][h] == -INFINITY) ? 0.f : __expf(sm_m[w][h] - mm);
            ll += sm_l[w][h] * f;
            a += sm_acc[w][h][d] * f;
        }
        if (nsplit == 1) {
            float o = ll > 0.f ? a / ll : 0.f;
            size_t col = (size_t)(kvh * G + h) * HD + d;
            if (p.gate_off >= 0) o *= sigmoid_f(__half2float(p.q[(size_t)r * p.ldq + p.gate_off + col]));
            p.out[(size_t)r * p.ldo + col] = __float2half(o);
        } else {
            my[h * (HD + 2) + d] = a;
            if (d == 0) { my[h * (HD + 2) + HD] = mm; my[h * (HD + 2) + HD + 1] = ll; }
        }
    }
    if (nsplit == 1) return;
    // ---- merge the splits: last CTA of this (row, kv head)
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int old = atomicAdd(&p.counters[r * p.nkv + kvh], 1);
        s_last = (old == nsplit - 1);
        if (s_last) p.counters[r * p.nkv + kvh] = 0;
        __threadfence();
    }
    __syncthreads();
    if (!s_last) return;
    const float* all = p.scratch + (((size_t)r * p.nkv + kvh) * splits_orig) * G * (HD + 2);
    // phase 1: per (split, head) rescale factors, one round trip
    for (int idx = tid; idx < nsplit * G; idx += ATT_THREADS) {
        int s = idx / G, h = idx % G;
        const float* e = &all[(size_t)(s * G + h) * (HD + 2)];
        sm_f[s][h] = ld_cg_f32(e + HD);                 // max of split s
        sm_acc[0][h][s] = ld_cg_f32(e + HD + 1);        // its sum (sm_acc is free by now)
    }
    __syncthreads();
    if (tid < G) {
        float mm = -INFINITY;
        for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, sm_f[s][tid]);
        float ll = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            float f = (sm_f[s][tid] == -INFINITY) ? 0.f : __expf(sm_f[s][tid] - mm);
            ll += sm_acc[0][tid][s] * f;
            sm_f[s][tid] = f;
        }
        sm_linv[tid] = ll > 0.f ? 1.f / ll : 0.f;
    }
    __syncthreads();
    // phase 2: weighted sum of the partial outputs; loads of several outputs are in flight together
#pragma unroll 4
    for (int i = tid; i < G * HD; i += ATT_THREADS) {
        int h = i / HD, d = i % HD;
        float a = 0.f;
        for (int s = 0; s < nsplit; ++s) a += ld_cg_f32(&all[(size_t)(s * G + h) * (HD + 2) + d]) * sm_f[s][h];
        float o = a * sm_linv[h];
        size_t col = (size_t)(kvh * G + h) * HD + d;
        if (p.gate_off >= 0) o *= sigmoid_f(__half2float(p.q[(size_t)r * p.ldq + p.gate_off + col]));
        p.out[(size_t)r * p.ldo + col] = __float2half(o);
    }
}

B2_API int b2_decode_attn(const AttnParams* p, int hd, cudaStream_t s) {
    if (p->nq % p->nkv || p->nq / p->nkv > ATT_MAX_G || p->splits < 1 || p->splits > 32) return cudaErrorInvalidValue;
    dim3 grid(p->nkv, p->n_rows, p->splits);
    if (hd == 256) return launch_pdl(decode_attn_kernel<256>, grid, dim3(ATT_THREADS), 0, s, *p);
    if (hd == 128) return launch_pdl(decode_attn_kernel<128>, grid, dim3(ATT_THREADS), 0, s, *p);
    if (hd == 64) return launch_pdl(decode_attn_kernel<64>, grid, dim3(ATT_THREADS), 0, s, *p);
    return cudaErrorInvalidValue;
}
B2_API int b2_sizeof_attn_params() { return (int)sizeof(AttnParams); }
