// Gated DeltaNet recurrent step (decode, chain verification, token-serial prefill).
//
// Per value head: causal conv1d(k=4)+SiLU on q,k,v -> L2-normalise q,k ->
// decay = exp(-exp(A_log) softplus(a+dt_bias)), beta = sigmoid(b) ->
//   S <- decay S;  delta = (v - S^T k) beta;  S <- S + k (x) delta;  y = S^T q
// -> y / rms(y) * norm_w * silu(z).  Same math as the reference's fused kernel
// and its CPU oracle (reference: src/kernels/deltanet_v3.hip:70-243,
// src/inference/engine.py:2094-2206); the conv-state shift that the reference
// runs as a second kernel (deltanet_v3.hip:54-65) is folded in.
//
// B200 mapping: the [dk x dv] fp32 state of a head is split by columns over a
// thread-block cluster of dv/32 CTAs (columns evolve independently), which
// gives 4x more CTAs than heads; the only cross-column quantity, sum(y^2) of
// the gated RMSNorm, is exchanged through distributed shared memory.  Each CTA
// keeps a private copy of the conv history of the channels it consumes, so no
// CTA reads history another CTA is shifting.  The state stays in registers
// while a sequence's rows (1 for decode, n for a draft chain or a prompt) are
// consumed in order: one HBM read and one write of the state per launch.
// The tiny a/b projections (2 rows of length hidden per head) can be computed
// in-kernel from the normalised activations, saving a launch.
#include <cooperative_groups.h>
#include "kernels.cuh"
namespace cg = cooperative_groups;

#define DN_THREADS 256
#define DN_COLS 32


template <int DK, int DV>
__global__ void __launch_bounds__(DN_THREADS) deltanet_step_kernel(const DeltaParams p) {
    constexpr int CB = DV / DN_COLS;
    constexpr int RPT = DK / 8;                  // state rows per thread
    constexpr int NCH = 2 * DK + DN_COLS;        // conv channels this CTA consumes
    cg::cluster_group cluster = cg::this_cluster();
    pdl_launch_dependents();
    const int cb = blockIdx.x, j = blockIdx.y, si = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, kr = tid >> 5, vcol = lane;
    const int kh = j / (p.nv / p.nk);
    const int r0 = p.seq_rows[si], r1 = p.seq_rows[si + 1];
    if (r0 >= r1) { return; }                    // uniform over the whole cluster
    const int seq = p.rows[r0].seq;

    __shared__ float hist[NCH][3];
    __shared__ float cw[NCH][4];
    __shared__ float cq[DK], ck[DK], cv[DN_COLS];
    __shared__ float red_m[8][DN_COLS], red_q[8][DN_COLS];
    __shared__ float red32[32];
    __shared__ float cl_ss[2];

    // channel id (in the q|k|v conv layout) of local channel c
    auto chan = [&](int c) -> int {
        if (c < DK) return kh * DK + c;
        if (c < 2 * DK) return p.nk * DK + kh * DK + (c - DK);
        return 2 * p.nk * DK + j * DV + cb * DN_COLS + (c - 2 * DK);
    };
    auto proj_col = [&](int c) -> int {
        if (c < DK) return p.off_q + kh * DK + c;
        if (c < 2 * DK) return p.off_k + kh * DK + (c - DK);
        return p.off_v + j * DV + cb * DN_COLS + (c - 2 * DK);
    };
    __half* my_hist = p.conv_state + ((((size_t)seq * p.nv + j) * CB + cb) * NCH) * 3;
    for (int c = tid; c < NCH; c += DN_THREADS) {
#pragma unroll
        for (int t = 0; t < 3; ++t) hist[c][t] = __half2float(my_hist[c * 3 + t]);
        const __half* w = p.conv_w + (size_t)chan(c) * 4;
#pragma unroll
        for (int t = 0; t < 4; ++t) cw[c][t] = __half2float(w[t]);
    }
    float S[RPT];
    float* sp = p.state + (((size_t)seq * p.nv + j) * DK) * DV + cb * DN_COLS + vcol;
#pragma unroll
    for (int i = 0; i < RPT; ++i) S[i] = sp[(size_t)(kr + 8 * i) * DV];
    const float neg_expA = -__expf(p.A_log[j]);
    const float dtb = __half2float(p.dt_bias[j]);
    const float nw = __half2float(p.norm_w[cb * DN_COLS + vcol]);
    __syncthreads();

    for (int r = r0; r < r1; ++r) {
        const __half* pr = p.proj + (size_t)r * p.ld;
        // ---- phase A (no barrier inside): conv + SiLU of this CTA's channels, partial sums of the
        // a/b projections.  With a lazily normalised input the 1/rms factor is applied to the
        // finished dot products, so nothing here waits on it.
        float sa = 0.f, sb = 0.f;
        const bool inkernel_ab = p.off_a < 0;
        if (inkernel_ab) {
            const __half* wa = p.wa + (size_t)j * p.H;
            const __half* wb = p.wb + (size_t)j * p.H;
            if (p.ln.h) {
                const float* hr = p.ln.h + (size_t)r * p.ln.H;
                for (int i = tid * 2; i < p.H; i += DN_THREADS * 2) {
                    float2 hv = *(const float2*)(hr + i);
                    float2 ww = __half22float2(*(const __half2*)(p.ln.w + i));
                    float2 av = __half22float2(*(const __half2*)(wa + i));
                    float2 bv = __half22float2(*(const __half2*)(wb + i));
                    float x0 = hv.x * ww.x, x1 = hv.y * ww.y;
                    sa += x0 * av.x + x1 * av.y;
                    sb += x0 * bv.x + x1 * bv.y;
                }
            } else {
                const __half* x = p.xn + (size_t)r * p.ldx;
                for (int i = tid * 2; i < p.H; i += DN_THREADS * 2) {
                    float2 xv = __half22float2(*(const __half2*)(x + i));
                    float2 av = __half22float2(*(const __half2*)(wa + i));
                    float2 bv = __half22float2(*(const __half2*)(wb + i));
                    sa += xv.x * av.x + xv.y * av.y;
                    sb += xv.x * bv.x + xv.y * bv.y;
                }
            }
            sa = warp_sum(sa);
            sb = warp_sum(sb);
            if (lane == 0) { red_m[kr][0] = sa; red_m[kr][1] = sb; }
        }
        for (int c = tid; c < NCH; c += DN_THREADS) {
            float x = __half2float(pr[proj_col(c)]);
            float o = hist[c][0] * cw[c][0] + hist[c][1] * cw[c][1] + hist[c][2] * cw[c][2] + x * cw[c][3];
            hist[c][0] = hist[c][1]; hist[c][1] = hist[c][2]; hist[c][2] = x;
            o = silu_f(o);
            if (c < DK) cq[c] = o; else if (c < 2 * DK) ck[c - DK] = o; else cv[c - 2 * DK] = o;
        }
        __syncthreads();
        // ---- phase B: warps 0..2 the q/k norms and q.k, warp 3 the a/b inputs
        if (kr < 3) {
            float s = 0.f;
            for (int i = lane; i < DK; i += 32) {
                float a = (kr == 1) ? ck[i] : cq[i], b = (kr == 0) ? cq[i] : ck[i];
                s += a * b;                      // kr0: q.q  kr1: k.k  kr2: q.k
            }
            s = warp_sum(s);
            if (lane == 0) red32[kr] = s;
        } else if (kr == 3) {
            float a_in, b_in;
            if (inkernel_ab) {
                float inv = p.ln.h ? lazy_inv_rms(p.ln, r, lane) : 1.f;
                float ta = 0.f, tb = 0.f;
#pragma unroll
                for (int w = 0; w < 8; ++w) { ta += red_m[w][0]; tb += red_m[w][1]; }
                // the unfused path rounds the projection output to fp16: keep that rounding
                a_in = __half2float(__float2half(ta * inv));
                b_in = __half2float(__float2half(tb * inv));
            } else {
                a_in = __half2float(pr[p.off_a + j]);
                b_in = __half2float(pr[p.off_b + j]);
            }
            if (lane == 0) { red32[3] = a_in; red32[4] = b_in; }
        }
        __syncthreads();
        const float invq = rsqrtf(red32[0] + 1e-6f) * rsqrtf((float)DK);
        const float invk = rsqrtf(red32[1] + 1e-6f);
        const float kq = red32[2] * invq * invk;
        const float a_in = red32[3], b_in = red32[4];
        float gl = neg_expA * (a_in + dtb > 20.f ? a_in + dtb : log1pf(__expf(a_in + dtb)));
        gl = fmaxf(gl, -20.f);
        const float decay = __expf(gl);
        const float beta = sigmoid_f(b_in);
        // ---- phase C: single pass over the state slice: m = S^T k, sq = S^T q
        float mp = 0.f, qp = 0.f;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            mp = fmaf(S[i], ck[kr + 8 * i], mp);
            qp = fmaf(S[i], cq[kr + 8 * i], qp);
        }
        red_m[kr][vcol] = mp * invk;
        red_q[kr][vcol] = qp * invq;
        __syncthreads();
        float mm = 0.f, sq = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) { mm += red_m[w][vcol]; sq += red_q[w][vcol]; }
        const float delta = (cv[vcol] - decay * mm) * beta;
        const float y = decay * sq + delta * kq;
#pragma unroll
        for (int i = 0; i < RPT; ++i) S[i] = decay * S[i] + ck[kr + 8 * i] * invk * delta;
        // ---- gated RMSNorm over the head's dv outputs (dv/32 CTAs of the cluster)
        float ss = warp_sum(y * y);              // every warp holds the same y per column
        const int slot = (r - r0) & 1;
        if (tid == 0) cl_ss[slot] = ss;
        cluster.sync();
        float tot = 0.f;
#pragma unroll
        for (int c = 0; c < CB; ++c) tot += *cluster.map_shared_rank(&cl_ss[slot], c);
        if (kr == 0) {
            float z = __half2float(pr[p.off_z + j * DV + cb * DN_COLS + vcol]);
            float o = y * rsqrtf(tot / (float)DV + p.eps) * nw * silu_f(z);
            p.out[(size_t)r * p.ldo + j * DV + cb * DN_COLS + vcol] = __float2half(o);
        }
        // the cluster barrier above also orders this row's shared-memory reads before the next row's writes
    }
    cluster.sync();                              // no CTA leaves while a peer may still read its shared memory
    if (!p.commit) return;
#pragma unroll
    for (int i = 0; i < RPT; ++i) sp[(size_t)(kr + 8 * i) * DV] = S[i];
    for (int c = tid; c < NCH; c += DN_THREADS)
#pragma unroll
        for (int t = 0; t < 3; ++t) my_hist[c * 3 + t] = __float2half(hist[c][t]);
}

template <int DK, int DV>
static int launch_delta(const DeltaParams* p, cudaStream_t s) {
    constexpr int CB = DV / DN_COLS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(CB, p->nv, p->n_seqs);
    cfg.blockDim = dim3(DN_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CB;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, deltanet_step_kernel<DK, DV>, *p);
}

B2_API int b2_deltanet_step(const DeltaParams* p, int dk, int dv, cudaStream_t s) {
    if (p->nv % p->nk) return cudaErrorInvalidValue;
    if (dk == 128 && dv == 128) return launch_delta<128, 128>(p, s);
    if (dk == 64 && dv == 64) return launch_delta<64, 64>(p, s);
    return cudaErrorInvalidValue;
}
B2_API int b2_sizeof_delta_params() { return (int)sizeof(DeltaParams); }
B2_API int b2_delta_conv_channels(int dk) { return 2 * dk + DN_COLS; }

// ===========================================================================
// Chunked Gated DeltaNet scan (prefill, long draft chains).
//
// The reference has no chunked form: its prefill loops the decode kernel token by token
// (reference: src/inference/engine.py:3141-3161).  Here a sequence is consumed in chunks of
// 64 rows.  With G_i the running sum of the log-decays inside a chunk and S0 the state at its
// start:
//     A[i][j] = beta_i exp(G_i-G_j) (k_i.k_j)  (j <  i)      W[i][j] = exp(G_i-G_j) (q_i.k_j)  (j <= i)
//     (I + A) U = beta (V - exp(G) K S0)                     (forward substitution, blocked by 8 rows)
//     Y  = exp(G) Q S0 + W U
//     S' = exp(G_C) S0 + (exp(G_C-G) K)^T U
// Same decomposition as the step kernel: a cluster of dv/32 CTAs per value head, each owning
// 32 state columns (columns never interact except through sum(y^2) of the gated RMSNorm,
// which is exchanged through distributed shared memory once per chunk).  All matrices of a
// chunk live in shared memory in fp32; the state slice stays in registers across chunks.
// ===========================================================================
#define DC_C 64                  // rows per chunk
#define DC_LDK(DK) ((DK) + 4)    // padded row stride of the q/k tiles
#define DC_LDA (DC_C + 4)

template <int DK, int DV>
__global__ void __launch_bounds__(DN_THREADS, 1) deltanet_chunk_kernel(const DeltaParams p, const __half* __restrict__ ab, int ld_ab) {
    constexpr int CB = DV / DN_COLS;
    constexpr int RPT = DK / 8;
    constexpr int NCH = 2 * DK + DN_COLS;
    constexpr int LDK = DC_LDK(DK);
    cg::cluster_group cluster = cg::this_cluster();
    pdl_launch_dependents();
    const int cb = blockIdx.x, j = blockIdx.y, si = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, kr = tid >> 5, vcol = lane;
    const int kh = j / (p.nv / p.nk);
    const int r0 = p.seq_rows[si], r1 = p.seq_rows[si + 1];
    if (r0 >= r1) return;
    const int seq = p.rows[r0].seq;

    extern __shared__ __align__(16) float dsm[];
    float* Qs = dsm;                          // [C][LDK]
    float* Ks = Qs + DC_C * LDK;              // [C][LDK]
    float* Us = Ks + DC_C * LDK;              // [C][32]  v -> b -> u (in place)
    float* QSs = Us + DC_C * DN_COLS;         // [C][32]  exp(G) Q S0
    float* Ys = QSs + DC_C * DN_COLS;         // [C][32]
    float* As = Ys + DC_C * DN_COLS;          // [C][LDA]
    float* Ws = As + DC_C * DC_LDA;           // [C][LDA]
    float* S0s = Ws + DC_C * DC_LDA;          // [DK][32]
    float* hist = S0s + DK * DN_COLS;         // [NCH][3]
    float* cw = hist + NCH * 3;               // [NCH][4]
    float* Gs = cw + NCH * 4;                 // [C] running log-decay
    float* bs = Gs + DC_C;                    // [C] beta
    float* gs = bs + DC_C;                    // [C] log-decay per row
    float* cl_ss = gs + DC_C;                 // [2][C]
    __half* Xr = (__half*)(cl_ss + 2 * DC_C);  // [C+3][NCH] raw conv inputs of the chunk (3 history rows first)

    auto chan = [&](int c) -> int {
        if (c < DK) return kh * DK + c;
        if (c < 2 * DK) return p.nk * DK + kh * DK + (c - DK);
        return 2 * p.nk * DK + j * DV + cb * DN_COLS + (c - 2 * DK);
    };
    auto proj_col = [&](int c) -> int {
        if (c < DK) return p.off_q + kh * DK + c;
        if (c < 2 * DK) return p.off_k + kh * DK + (c - DK);
        return p.off_v + j * DV + cb * DN_COLS + (c - 2 * DK);
    };
    __half* my_hist = p.conv_state + ((((size_t)seq * p.nv + j) * CB + cb) * NCH) * 3;
    for (int c = tid; c < NCH; c += DN_THREADS) {
#pragma unroll
        for (int t = 0; t < 3; ++t) hist[c * 3 + t] = __half2float(my_hist[c * 3 + t]);
        const __half* w = p.conv_w + (size_t)chan(c) * 4;
#pragma unroll
        for (int t = 0; t < 4; ++t) cw[c * 4 + t] = __half2float(w[t]);
    }
    float S[RPT];
    float* sp = p.state + (((size_t)seq * p.nv + j) * DK) * DV + cb * DN_COLS + vcol;
#pragma unroll
    for (int i = 0; i < RPT; ++i) S[i] = sp[(size_t)(kr + 8 * i) * DV];
    const float neg_expA = -__expf(p.A_log[j]);
    const float dtb = __half2float(p.dt_bias[j]);
    const float nw = __half2float(p.norm_w[cb * DN_COLS + vcol]);
    const float qscale = rsqrtf((float)DK);
    __syncthreads();

    // raw-tile staging: 16-byte cp.async pieces; rows before the sequence start come from the saved history,
    // rows past its end are zero
    auto stage_raw = [&](int rb_) {
        constexpr int PPR = NCH / 8;                       // 16-byte pieces per row
        for (int idx = tid; idx < (DC_C + 3) * PPR; idx += DN_THREADS) {
            const int row = idx / PPR, pc = idx % PPR;
            const int c = pc * 8;
            const int ri = rb_ - 3 + row;
            __half* dst = Xr + row * NCH + c;
            if (ri >= r0 && ri < r1) {
                cp_async16(dst, p.proj + (size_t)ri * p.ld + proj_col(c));
            } else if (ri < r0) {
#pragma unroll
                for (int e = 0; e < 8; ++e) dst[e] = __float2half(hist[(c + e) * 3 + (ri - r0 + 3)]);
            } else {
                *(uint4*)dst = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        cp_async_commit();
    };
    stage_raw(r0);

    int chunk_idx = 0;
    for (int rb = r0; rb < r1; rb += DC_C, ++chunk_idx) {
        const int Ce = min(DC_C, r1 - rb);
        // ---- P1: causal conv + SiLU from the raw tile staged in shared memory by cp.async (the
        // copy for this chunk was issued while the previous chunk was being processed)
        cp_async_wait<0>();
        __syncthreads();
        for (int item = tid; item < NCH * (DC_C / 8); item += DN_THREADS) {
            const int c = item % NCH, i0 = (item / NCH) * 8;
            const float w0 = cw[c * 4 + 0], w1 = cw[c * 4 + 1], w2 = cw[c * 4 + 2], w3 = cw[c * 4 + 3];
            float x0 = __half2float(Xr[(i0 + 0) * NCH + c]), x1 = __half2float(Xr[(i0 + 1) * NCH + c]);
            float x2 = __half2float(Xr[(i0 + 2) * NCH + c]);
            float* dst = (c < DK) ? Qs + c : (c < 2 * DK) ? Ks + (c - DK) : Us + (c - 2 * DK);
            const int ldd = (c < 2 * DK) ? LDK : DN_COLS;
#pragma unroll
            for (int i = i0; i < i0 + 8; ++i) {
                const float x3 = __half2float(Xr[(i + 3) * NCH + c]);
                const float acc = x0 * w0 + x1 * w1 + x2 * w2 + x3 * w3;
                dst[i * ldd] = (i < Ce) ? silu_f(acc) : 0.f;
                x0 = x1; x1 = x2; x2 = x3;
            }
        }
        if (tid < DC_C) {
            float gl = 0.f, beta = 0.f;
            if (tid < Ce) {
                const __half* abr = ab + (size_t)(rb + tid) * ld_ab;
                float a_in = __half2float(abr[j]), b_in = __half2float(abr[p.nv + j]);
                float sp_ = a_in + dtb;
                gl = fmaxf(neg_expA * (sp_ > 20.f ? sp_ : log1pf(__expf(sp_))), -20.f);
                beta = sigmoid_f(b_in);
            }
            gs[tid] = gl;
            bs[tid] = beta;
        }
        __syncthreads();
        if (rb + DC_C < r1) stage_raw(rb + DC_C);          // flies while this chunk is processed
        // ---- P2: L2-normalise q and k rows, running log-decay
        for (int i = kr; i < DC_C; i += 8) {
            float qq = 0.f, kk = 0.f;
            for (int k = lane; k < DK; k += 32) { float a = Qs[i * LDK + k], b = Ks[i * LDK + k]; qq += a * a; kk += b * b; }
            qq = warp_sum(qq); kk = warp_sum(kk);
            const float iq = rsqrtf(qq + 1e-6f) * qscale, ik = rsqrtf(kk + 1e-6f);
            for (int k = lane; k < DK; k += 32) { Qs[i * LDK + k] *= iq; Ks[i * LDK + k] *= ik; }
        }
        if (tid == 0) {
            float run = 0.f;
            for (int i = 0; i < DC_C; ++i) { run += gs[i]; Gs[i] = run; }
        }
        // state slice to shared memory for the S0 products
#pragma unroll
        for (int i = 0; i < RPT; ++i) S0s[(kr + 8 * i) * DN_COLS + vcol] = S[i];
        __syncthreads();
        // ---- P3: A and W (lower triangle), 4x4 register tiles
        {
            const int ti = tid >> 4, tj = tid & 15;
            if (tj <= ti) {
                float kk[4][4], qk[4][4];
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b) kk[a][b] = qk[a][b] = 0.f;
                for (int k = 0; k < DK; k += 4) {
                    float4 kr4[4], qr4[4], kc4[4];
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
                        kr4[a] = *(const float4*)&Ks[(4 * ti + a) * LDK + k];
                        qr4[a] = *(const float4*)&Qs[(4 * ti + a) * LDK + k];
                        kc4[a] = *(const float4*)&Ks[(4 * tj + a) * LDK + k];
                    }
#pragma unroll
                    for (int a = 0; a < 4; ++a)
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            kk[a][b] += kr4[a].x * kc4[b].x + kr4[a].y * kc4[b].y + kr4[a].z * kc4[b].z + kr4[a].w * kc4[b].w;
                            qk[a][b] += qr4[a].x * kc4[b].x + qr4[a].y * kc4[b].y + qr4[a].z * kc4[b].z + qr4[a].w * kc4[b].w;
                        }
                }
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        const int i = 4 * ti + a, jj = 4 * tj + b;
                        const float dec = (jj <= i) ? __expf(Gs[i] - Gs[jj]) : 0.f;
                        As[i * DC_LDA + jj] = (jj < i) ? bs[i] * dec * kk[a][b] : 0.f;
                        Ws[i * DC_LDA + jj] = dec * qk[a][b];
                    }
            }
        }
        // ---- P4: K S0 and Q S0; b = beta (v - exp(G) K S0) in place of v
        {
            float ak[8], aq[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) ak[u] = aq[u] = 0.f;
            for (int k = 0; k < DK; k += 4) {
                const float s0 = S0s[(k + 0) * DN_COLS + vcol], s1 = S0s[(k + 1) * DN_COLS + vcol];
                const float s2 = S0s[(k + 2) * DN_COLS + vcol], s3 = S0s[(k + 3) * DN_COLS + vcol];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = kr + 8 * u;
                    const float4 k4 = *(const float4*)&Ks[i * LDK + k], q4 = *(const float4*)&Qs[i * LDK + k];
                    ak[u] += k4.x * s0 + k4.y * s1 + k4.z * s2 + k4.w * s3;
                    aq[u] += q4.x * s0 + q4.y * s1 + q4.z * s2 + q4.w * s3;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = kr + 8 * u;
                const float eg = __expf(Gs[i]);
                Us[i * DN_COLS + vcol] = bs[i] * (Us[i * DN_COLS + vcol] - eg * ak[u]);
                QSs[i * DN_COLS + vcol] = eg * aq[u];
            }
        }
        __syncthreads();
        // ---- P5: (I + A) U = B by forward substitution, 8 rows per block: every warp first removes
        // the contribution of all earlier blocks from its row, then warp 0 finishes the 8x8 triangle
        for (int blk = 0; blk < DC_C / 8; ++blk) {
            const int i = 8 * blk + kr;
            float acc = Us[i * DN_COLS + vcol];
            for (int jj = 0; jj < 8 * blk; ++jj) acc = fmaf(-As[i * DC_LDA + jj], Us[jj * DN_COLS + vcol], acc);
            Us[i * DN_COLS + vcol] = acc;
            __syncthreads();
            if (kr == 0) {
#pragma unroll
                for (int a = 1; a < 8; ++a) {
                    const int ia = 8 * blk + a;
                    float t = Us[ia * DN_COLS + vcol];
#pragma unroll
                    for (int b = 0; b < 8; ++b)
                        if (b < a) t = fmaf(-As[ia * DC_LDA + 8 * blk + b], Us[(8 * blk + b) * DN_COLS + vcol], t);
                    Us[ia * DN_COLS + vcol] = t;
                }
            }
            __syncthreads();
        }
        // ---- P6: Y = exp(G) Q S0 + W U, partial sum of squares per row
        const int slot = chunk_idx & 1;
#pragma unroll 1
        for (int u = 0; u < 8; ++u) {
            const int i = kr + 8 * u;
            float y = QSs[i * DN_COLS + vcol];
            for (int jj = 0; jj <= i; ++jj) y = fmaf(Ws[i * DC_LDA + jj], Us[jj * DN_COLS + vcol], y);
            Ys[i * DN_COLS + vcol] = y;
            float ss = warp_sum(y * y);
            if (lane == 0) cl_ss[slot * DC_C + i] = ss;
        }
        // ---- P7: S' = exp(G_C) S0 + (exp(G_C - G) K)^T U   (state slice in registers)
        {
            const float gC = Gs[DC_C - 1];
            const float egC = __expf(gC);
#pragma unroll
            for (int i2 = 0; i2 < RPT; ++i2) S[i2] *= egC;
            for (int i = 0; i < Ce; ++i) {
                const float u = Us[i * DN_COLS + vcol] * __expf(gC - Gs[i]);
#pragma unroll
                for (int i2 = 0; i2 < RPT; ++i2) S[i2] = fmaf(Ks[i * LDK + kr + 8 * i2], u, S[i2]);
            }
        }
        cluster.sync();
        // ---- gated RMSNorm across the head's column blocks, output
#pragma unroll 1
        for (int u = 0; u < 8; ++u) {
            const int i = kr + 8 * u;
            if (i < Ce) {
                float tot = 0.f;
#pragma unroll
                for (int c = 0; c < CB; ++c) tot += cluster.map_shared_rank(cl_ss, c)[slot * DC_C + i];
                const int r = rb + i;
                const float z = __half2float(p.proj[(size_t)r * p.ld + p.off_z + j * DV + cb * DN_COLS + vcol]);
                const float o = Ys[i * DN_COLS + vcol] * rsqrtf(tot / (float)DV + p.eps) * nw * silu_f(z);
                p.out[(size_t)r * p.ldo + j * DV + cb * DN_COLS + vcol] = __float2half(o);
            }
        }
        __syncthreads();
    }
    cluster.sync();
    if (!p.commit) return;
#pragma unroll
    for (int i = 0; i < RPT; ++i) sp[(size_t)(kr + 8 * i) * DV] = S[i];
    // last three raw conv inputs (older history shifts in when the sequence was shorter than 3 rows)
    const int n = r1 - r0;
    for (int c = tid; c < NCH; c += DN_THREADS) {
        const int col = proj_col(c);
#pragma unroll
        for (int t = 0; t < 3; ++t) {
            const int ri = r1 - 3 + t;
            float x = (ri >= r0) ? __half2float(p.proj[(size_t)ri * p.ld + col]) : hist[c * 3 + (ri - r0 + 3)];
            my_hist[c * 3 + t] = __float2half(x);
        }
    }
    (void)n;
}

template <int DK, int DV>
static int launch_delta_chunk(const DeltaParams* p, const void* ab, int ld_ab, cudaStream_t s) {
    constexpr int CB = DV / DN_COLS;
    constexpr int NCH = 2 * DK + DN_COLS;
    size_t smem = (size_t)(2 * DC_C * DC_LDK(DK) + 3 * DC_C * DN_COLS + 2 * DC_C * DC_LDA + DK * DN_COLS + NCH * 7 +
                           3 * DC_C + 2 * DC_C) * sizeof(float) + (size_t)(DC_C + 3) * NCH * sizeof(__half);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(deltanet_chunk_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(CB, p->nv, p->n_seqs);
    cfg.blockDim = dim3(DN_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CB;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, deltanet_chunk_kernel<DK, DV>, *p, (const __half*)ab, ld_ab);
}

// ab: [rows][ld_ab] fp16 with a at column head and b at column nv + head.
B2_API int b2_deltanet_chunk(const DeltaParams* p, const void* ab, int ld_ab, int dk, int dv, cudaStream_t s) {
    if (p->nv % p->nk || !ab) return cudaErrorInvalidValue;
    if (dk == 128 && dv == 128) return launch_delta_chunk<128, 128>(p, ab, ld_ab, s);
    if (dk == 64 && dv == 64) return launch_delta_chunk<64, 64>(p, ab, ld_ab, s);
    return cudaErrorInvalidValue;
}

// a/b projections for many rows: ab[r][o] = x[r] . w[o], o < n_out (tiny dense weights).
__global__ void __launch_bounds__(256) ab_proj_kernel(const __half* __restrict__ x, int ldx, const __half* __restrict__ wa,
                                                      const __half* __restrict__ wb, int nv, int H,
                                                      __half* __restrict__ ab, int ld_ab) {
    extern __shared__ __align__(16) __half xs[];
    pdl_launch_dependents();
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid * 8; i < H; i += 256 * 8) *(uint4*)(xs + i) = *(const uint4*)(x + (size_t)r * ldx + i);
    __syncthreads();
    for (int o = warp; o < 2 * nv; o += 8) {
        const __half* w = (o < nv) ? wa + (size_t)o * H : wb + (size_t)(o - nv) * H;
        float acc = 0.f;
        for (int i = lane * 8; i < H; i += 256) {
            uint4 wv = *(const uint4*)(w + i), xv = *(const uint4*)(xs + i);
            const __half2* w2 = (const __half2*)&wv; const __half2* x2 = (const __half2*)&xv;
#pragma unroll
            for (int q = 0; q < 4; ++q) { float2 a = __half22float2(w2[q]), b = __half22float2(x2[q]); acc += a.x * b.x + a.y * b.y; }
        }
        acc = warp_sum(acc);
        if (lane == 0) ab[(size_t)r * ld_ab + o] = __float2half(acc);
    }
}
B2_API int b2_ab_proj(const void* x, int ldx, const void* wa, const void* wb, int nv, int H, void* ab, int ld_ab,
                      int rows, cudaStream_t s) {
    if (H % 8) return cudaErrorInvalidValue;
    ab_proj_kernel<<<rows, 256, (size_t)H * 2, s>>>((const __half*)x, ldx, (const __half*)wa, (const __half*)wb, nv, H,
                                                    (__half*)ab, ld_ab);
    return cudaGetLastError();
}
