// Small memory-bound kernels of the decode and prefill paths: row set-up,
// embedding gather + first RMSNorm, RMSNorm / residual+RMSNorm, per-head
// QK-norm + partial RoPE + KV-cache write, SiLU*mul, sigmoid*mul, residual add.
//
// They replace the reference's elementwise_v2/v3, batched_rmsnorm, rope_v2,
// qknorm_rope, qknorm_rope_cachew and sigmoid_mul kernels (reference:
// src/kernels/elementwise_v3.hip:28-330, batched_rmsnorm.hip:27,
// rope_v2.hip:40, qknorm_rope.hip:55, qknorm_rope_cachew.hip:52,
// sigmoid_mul.hip:10).  Differences: positions, cache slots and sequence ids
// come from a device-resident RowMeta array, so a captured CUDA graph replays
// unchanged; the residual stream is fp32.
#include "gemv.cuh"

// ---------------------------------------------------------------------------
// prepare_rows: fill RowMeta from the per-sequence state and a static template.
// tmpl[r] = {seq, depth, slot_offset, unused, mask}: pos = len+depth, slot = len+slot_offset.
// ---------------------------------------------------------------------------
// step_word (optional): the step's generation, advanced by 1024 here; kernels of the step derive tags that
// no earlier step used from it (csrc/gemv.cu, tagged split-K hand-off).
__global__ void prepare_rows_kernel(const RowMeta* __restrict__ tmpl, const SeqState* __restrict__ seqs,
                                    RowMeta* __restrict__ rows, int n, unsigned int* step_word) {
    pdl_launch_dependents();
    if (step_word && blockIdx.x == 0 && threadIdx.x == 0) *step_word += 1024u;
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n) return;
    RowMeta t = tmpl[r];
    int len = seqs[t.seq].len;
    RowMeta o;
    o.seq = t.seq;
    o.pos = len + t.pos;
    o.slot = len + t.slot;
    o.ctx = len + t.ctx;          // template ctx: extra visible slots (prefill row i sees i+1 new ones)
    o.mask = t.mask;
    rows[r] = o;
}

B2_API int b2_prepare_rows(const void* tmpl, const void* seqs, void* rows, int n, unsigned int* step_word, cudaStream_t s) {
    prepare_rows_kernel<<<(n + 63) / 64, 64, 0, s>>>((const RowMeta*)tmpl, (const SeqState*)seqs, (RowMeta*)rows, n, step_word);
    return cudaGetLastError();
}

// advance: len += add[seq] for every sequence (after a step has been committed)
__global__ void advance_kernel(SeqState* seqs, const int* __restrict__ add, int n, int add_const) {
    pdl_launch_dependents();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) seqs[i].len += add ? add[i] : add_const;
}
B2_API int b2_advance(void* seqs, const int* add, int n, int add_const, cudaStream_t s) {
    advance_kernel<<<(n + 63) / 64, 64, 0, s>>>((SeqState*)seqs, add, n, add_const);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// embed_rmsnorm: h[r] = embed[token], xn[r] = rmsnorm(h[r]) * w.  One CTA per row.
// token = row_tokens[r] if >= 0 else seqs[rows[r].seq].token.
// ---------------------------------------------------------------------------
__global__ void embed_rmsnorm_kernel(const __half* __restrict__ embed, const int* __restrict__ row_tokens,
                                     const RowMeta* __restrict__ rows, const SeqState* __restrict__ seqs,
                                     const __half* __restrict__ w, float* __restrict__ h,
                                     __half* __restrict__ xn, float* __restrict__ ss_part, int np,
                                     int H, float eps, int vocab) {
    __shared__ float red[32];
    pdl_launch_dependents();
    int r = blockIdx.x;
    int tok = row_tokens ? row_tokens[r] : -1;
    if (tok < 0) tok = seqs[rows[r].seq].token;
    tok = min(max(tok, 0), vocab - 1);
    const __half* e = embed + (size_t)tok * H;
    float ss = 0.f;
    for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
        float2 v = __half22float2(*(const __half2*)(e + i));
        *(float2*)(h + (size_t)r * H + i) = v;
        ss += v.x * v.x + v.y * v.y;
    }
    float tot = block_sum(ss, red);
    if (ss_part) for (int i = threadIdx.x; i < np; i += blockDim.x) ss_part[(size_t)r * np + i] = i ? 0.f : tot;
    if (!xn) return;
    float inv = rsqrtf(tot / (float)H + eps);
    for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
        float2 v = *(const float2*)(h + (size_t)r * H + i);
        float2 ww = __half22float2(*(const __half2*)(w + i));
        *(__half2*)(xn + (size_t)r * H + i) = __floats2half2_rn(v.x * inv * ww.x, v.y * inv * ww.y);
    }
}
B2_API int b2_embed_rmsnorm(const void* embed, const int* row_tokens, const void* rows, const void* seqs,
                            const void* w, float* h, void* xn, float* ss_part, int np, int n_rows, int H,
                            float eps, int vocab, cudaStream_t s) {
    embed_rmsnorm_kernel<<<n_rows, 256, 0, s>>>((const __half*)embed, row_tokens, (const RowMeta*)rows,
                                                (const SeqState*)seqs, (const __half*)w, h, (__half*)xn, ss_part, np,
                                                H, eps, vocab);
    return cudaGetLastError();
}

// Same for rows whose embeddings come from the caller (the reference's
// embedding-in interface): h = emb (fp16 or fp32 input), xn = rmsnorm(h)*w.
__global__ void load_rmsnorm_kernel(const __half* __restrict__ emb16, const float* __restrict__ emb32,
                                    const __half* __restrict__ w, float* __restrict__ h,
                                    __half* __restrict__ xn, float* __restrict__ ss_part, int np, int H, float eps) {
    __shared__ float red[32];
    int r = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = emb32 ? emb32[(size_t)r * H + i] : __half2float(emb16[(size_t)r * H + i]);
        h[(size_t)r * H + i] = v;
        ss += v * v;
    }
    float tot = block_sum(ss, red);
    if (ss_part) for (int i = threadIdx.x; i < np; i += blockDim.x) ss_part[(size_t)r * np + i] = i ? 0.f : tot;
    if (!xn) return;
    float inv = rsqrtf(tot / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        xn[(size_t)r * H + i] = __float2half(h[(size_t)r * H + i] * inv * __half2float(w[i]));
}
B2_API int b2_load_rmsnorm(const void* emb16, const float* emb32, const void* w, float* h, void* xn,
                           float* ss_part, int np, int n_rows, int H, float eps, cudaStream_t s) {
    load_rmsnorm_kernel<<<n_rows, 256, 0, s>>>((const __half*)emb16, emb32, (const __half*)w, h, (__half*)xn, ss_part, np, H, eps);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// rmsnorm / add_rmsnorm on the fp32 residual stream: h += delta (optional),
// xn = rmsnorm(h) * w.  One CTA per row.
// ---------------------------------------------------------------------------
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta32,
                                   const __half* __restrict__ delta16, const __half* __restrict__ w,
                                   __half* __restrict__ xn, float* __restrict__ xn32, int H, float eps) {
    __shared__ float red[32];
    int r = blockIdx.x;
    float* hr = h + (size_t)r * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = hr[i];
        if (delta32) v += delta32[(size_t)r * H + i];
        if (delta16) v += __half2float(delta16[(size_t)r * H + i]);
        if (delta32 || delta16) hr[i] = v;
        ss += v * v;
    }
    float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = hr[i] * inv * __half2float(w[i]);
        if (xn) xn[(size_t)r * H + i] = __float2half(v);
        if (xn32) xn32[(size_t)r * H + i] = v;
    }
}
// Same, for H % 4 == 0 and H <= 8192: the row is read once with 16-byte loads and kept in registers.
__global__ void __launch_bounds__(256) add_rmsnorm_vec_kernel(float* __restrict__ h, const float* __restrict__ delta32,
                                                              const __half* __restrict__ delta16,
                                                              const __half* __restrict__ w, __half* __restrict__ xn,
                                                              float* __restrict__ xn32, int H, float eps) {
    __shared__ float red[32];
    pdl_launch_dependents();
    const int r = blockIdx.x, n4 = H >> 2;
    float4* hr = (float4*)(h + (size_t)r * H);
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int i = threadIdx.x + 256 * u;
        if (i < n4) {
            float4 a = hr[i];
            if (delta32) { const float4 d = ((const float4*)(delta32 + (size_t)r * H))[i]; a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w; }
            if (delta16) {
                const uint2 d = ((const uint2*)(delta16 + (size_t)r * H))[i];
                const float2 d0 = __half22float2(*(const __half2*)&d.x), d1 = __half22float2(*(const __half2*)&d.y);
                a.x += d0.x; a.y += d0.y; a.z += d1.x; a.w += d1.y;
            }
            v[u] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int i = threadIdx.x + 256 * u;
        if (i < n4) {
            if (delta32 || delta16) hr[i] = v[u];
            const uint2 wv = ((const uint2*)w)[i];
            const float2 w0 = __half22float2(*(const __half2*)&wv.x), w1 = __half22float2(*(const __half2*)&wv.y);
            const float4 o = make_float4(v[u].x * inv * w0.x, v[u].y * inv * w0.y, v[u].z * inv * w1.x, v[u].w * inv * w1.y);
            if (xn) {
                const __half2 a = __floats2half2_rn(o.x, o.y), b = __floats2half2_rn(o.z, o.w);
                uint2 pk; pk.x = *(const uint32_t*)&a; pk.y = *(const uint32_t*)&b;
                ((uint2*)(xn + (size_t)r * H))[i] = pk;
            }
            if (xn32) ((float4*)(xn32 + (size_t)r * H))[i] = o;
        }
    }
}
B2_API int b2_add_rmsnorm(float* h, const float* delta32, const void* delta16, const void* w, void* xn,
                          float* xn32, int n_rows, int H, float eps, cudaStream_t s) {
    if (H % 4 == 0 && H <= 8192) {
        add_rmsnorm_vec_kernel<<<n_rows, 256, 0, s>>>(h, delta32, (const __half*)delta16, (const __half*)w,
                                                      (__half*)xn, xn32, H, eps);
        return cudaGetLastError();
    }
    add_rmsnorm_kernel<<<n_rows, 256, 0, s>>>(h, delta32, (const __half*)delta16, (const __half*)w,
                                              (__half*)xn, xn32, H, eps);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// qknorm_rope_cachew.  qkv[r] = [Q (nq*hd) | gate (nq*hd) | K (nkv*hd) | V (nkv*hd)] fp16.
// Q heads: RMSNorm * q_norm, RoPE on the first `rot` dims, written back in place.
// K heads: RMSNorm * k_norm, RoPE, written to the K cache at (seq, slot).
// V heads: copied to the V cache.  grid = (nq + 2*nkv, rows), block = hd.
// Cache layout per layer: [seq][max_seq][nkv][hd].
// ---------------------------------------------------------------------------
__global__ void qknorm_rope_cachew_kernel(__half* __restrict__ qkv, int ld, const RowMeta* __restrict__ rows,
                                          const __half* __restrict__ q_norm, const __half* __restrict__ k_norm,
                                          const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                          __half* __restrict__ kcache, __half* __restrict__ vcache,
                                          int nq, int nkv, int hd, int rot, int max_seq, int interleaved,
                                          float eps) {
    extern __shared__ float sv[];           // [hd]
    __shared__ float red[32];
    const int hidx = blockIdx.x, r = blockIdx.y, i = threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();                             // the in-projection's output
    const RowMeta rm = rows[r];
    __half* row = qkv + (size_t)r * ld;
    const size_t cache_off = (((size_t)rm.seq * max_seq + rm.slot) * nkv) * hd;
    if (hidx >= nq + nkv) {                 // V head: plain copy
        int kvh = hidx - nq - nkv;
        vcache[cache_off + (size_t)kvh * hd + i] = row[2 * nq * hd + nkv * hd + kvh * hd + i];
        return;
    }
    const bool is_q = hidx < nq;
    __half* src = is_q ? row + hidx * hd : row + 2 * nq * hd + (hidx - nq) * hd;
    const __half* nw = is_q ? q_norm : k_norm;
    float v = __half2float(src[i]);
    float inv = rsqrtf(block_sum(v * v, red) / (float)hd + eps);
    sv[i] = v * inv * __half2float(nw[i]);
    __syncthreads();
    float out = sv[i];
    if (i < rot) {
        const int half = rot >> 1;
        int pair, first;
        if (interleaved) { pair = i >> 1; first = !(i & 1); }
        else { pair = i % half; first = i < half; }
        float c = cos_tab[(size_t)rm.pos * half + pair], s = sin_tab[(size_t)rm.pos * half + pair];
        int j = interleaved ? (i ^ 1) : (first ? i + half : i - half);
        float other = sv[j];
        out = first ? sv[i] * c - other * s : other * s + sv[i] * c;
    }
    if (is_q) src[i] = __float2half(out);
    else kcache[cache_off + (size_t)(hidx - nq) * hd + i] = __float2half(out);
}
B2_API int b2_qknorm_rope_cachew(void* qkv, int ld, const void* rows, const void* q_norm, const void* k_norm,
                                 const float* cos_tab, const float* sin_tab, void* kcache, void* vcache,
                                 int n_rows, int nq, int nkv, int hd, int rot, int max_seq, int interleaved,
                                 float eps, cudaStream_t s) {
    dim3 grid(nq + 2 * nkv, n_rows);
    return launch_pdl(qknorm_rope_cachew_kernel, grid, dim3(hd), hd * sizeof(float), s,
                      (__half*)qkv, ld, (const RowMeta*)rows, (const __half*)q_norm, (const __half*)k_norm, cos_tab, sin_tab,
                      (__half*)kcache, (__half*)vcache, nq, nkv, hd, rot, max_seq, interleaved, eps);
}

// ---------------------------------------------------------------------------
// Plain elementwise ops (used where the op is not fused into a producer).
// ---------------------------------------------------------------------------
__global__ void silu_mul_kernel(const __half* __restrict__ gate, const __half* __restrict__ up,
                                __half* __restrict__ out, size_t n) {
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i + 1 < n) {
        float2 g = __half22float2(*(const __half2*)(gate + i)), u = __half22float2(*(const __half2*)(up + i));
        *(__half2*)(out + i) = __floats2half2_rn(silu_f(g.x) * u.x, silu_f(g.y) * u.y);
    } else if (i < n) {
        out[i] = __float2half(silu_f(__half2float(gate[i])) * __half2float(up[i]));
    }
}
B2_API int b2_silu_mul(const void* gate, const void* up, void* out, size_t n, cudaStream_t s) {
    size_t thr = (n + 1) / 2;
    silu_mul_kernel<<<(unsigned)((thr + 255) / 256), 256, 0, s>>>((const __half*)gate, (const __half*)up, (__half*)out, n);
    return cudaGetLastError();
}

// gate/up interleaved by 8 in one row of width 2F (the GEMM output layout): out[r][j]
__global__ void silu_mul_pair8_kernel(const __half* __restrict__ gu, int ld, __half* __restrict__ out, int ldo,
                                      int F, int rows) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * F) return;
    int r = idx / F, j = idx % F;
    const __half* row = gu + (size_t)r * ld + (j >> 3) * 16 + (j & 7);
    out[(size_t)r * ldo + j] = __float2half(silu_f(__half2float(row[0])) * __half2float(row[8]));
}
B2_API int b2_silu_mul_pair8(const void* gu, int ld, void* out, int ldo, int F, int rows, cudaStream_t s) {
    int n = rows * F;
    silu_mul_pair8_kernel<<<(n + 255) / 256, 256, 0, s>>>((const __half*)gu, ld, (__half*)out, ldo, F, rows);
    return cudaGetLastError();
}

__global__ void sigmoid_mul_kernel(__half* __restrict__ x, const __half* __restrict__ gate, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = __float2half(__half2float(x[i]) * sigmoid_f(__half2float(gate[i])));
}
B2_API int b2_sigmoid_mul(void* x, const void* gate, size_t n, cudaStream_t s) {
    sigmoid_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>((__half*)x, (const __half*)gate, n);
    return cudaGetLastError();
}

__global__ void residual_add_kernel(float* __restrict__ h, const float* __restrict__ d32,
                                    const __half* __restrict__ d16, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) h[i] += d32 ? d32[i] : __half2float(d16[i]);
}
B2_API int b2_residual_add(float* h, const float* d32, const void* d16, size_t n, cudaStream_t s) {
    residual_add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(h, d32, (const __half*)d16, n);
    return cudaGetLastError();
}

// h[r] += d32[r] (d32 may be null) and ss[r][0] = sum(h[r]^2), ss[r][1..np) = 0: what a consumer that
// normalises lazily (LazyNorm) expects from its producer.
__global__ void __launch_bounds__(256) residual_add_ss_kernel(float* __restrict__ h, const float* __restrict__ d32,
                                                              float* __restrict__ ss, int np, int H) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    float acc = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = h[(size_t)r * H + i];
        if (d32) { v += d32[(size_t)r * H + i]; h[(size_t)r * H + i] = v; }
        acc += v * v;
    }
    const float tot = block_sum(acc, red);
    if (ss) for (int i = threadIdx.x; i < np; i += blockDim.x) ss[(size_t)r * np + i] = i ? 0.f : tot;
}
B2_API int b2_residual_add_ss(float* h, const float* d32, float* ss, int np, int n_rows, int H, cudaStream_t s) {
    residual_add_ss_kernel<<<n_rows, 256, 0, s>>>(h, d32, ss, np, H);
    return cudaGetLastError();
}

__global__ void f32_to_f16_kernel(const float* __restrict__ a, __half* __restrict__ b, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) b[i] = __float2half(a[i]);
}
B2_API int b2_f32_to_f16(const float* a, void* b, size_t n, cudaStream_t s) {
    f32_to_f16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, (__half*)b, n);
    return cudaGetLastError();
}
