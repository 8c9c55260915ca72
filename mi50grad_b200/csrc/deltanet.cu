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
