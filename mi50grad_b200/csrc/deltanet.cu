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
#include <cstdlib>
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
    // The a/b projections' weights (times the norm weights of a lazily normalised input) do not depend on
    // this step either: the first DN_PRE pairs per thread wait in registers.
    constexpr int DN_PRE = 10;
    const bool inkernel_ab = p.off_a < 0;
    float2 pa[DN_PRE], pb[DN_PRE];
#pragma unroll
    for (int k = 0; k < DN_PRE; ++k) {
        pa[k] = pb[k] = make_float2(0.f, 0.f);
        const int i = tid * 2 + k * DN_THREADS * 2;
        if (inkernel_ab && i < p.H) {
            float2 av = __half22float2(*(const __half2*)(p.wa + (size_t)j * p.H + i));
            float2 bv = __half22float2(*(const __half2*)(p.wb + (size_t)j * p.H + i));
            if (p.ln.h) {
                const float2 ww = __half22float2(*(const __half2*)(p.ln.w + i));
                av.x *= ww.x; av.y *= ww.y; bv.x *= ww.x; bv.y *= ww.y;
            }
            pa[k] = av; pb[k] = bv;
        }
    }
    __syncthreads();
    // Everything above (conv history, state slice, weights) was left by earlier steps; what follows reads
    // this step's in-projection output and residual stream.
    pdl_wait();

    for (int r = r0; r < r1; ++r) {
        const __half* pr = p.proj + (size_t)r * p.ld;
        // ---- phase A (no barrier inside): conv + SiLU of this CTA's channels, partial sums of the
        // a/b projections.  With a lazily normalised input the 1/rms factor is applied to the
        // finished dot products, so nothing here waits on it.
        float sa = 0.f, sb = 0.f;
        if (inkernel_ab) {
            const __half* wa = p.wa + (size_t)j * p.H;
            const __half* wb = p.wb + (size_t)j * p.H;
            if (p.ln.h) {
                const float* hr = p.ln.h + (size_t)r * p.ln.H;
                float2 hv[DN_PRE];
#pragma unroll
                for (int k = 0; k < DN_PRE; ++k) {
                    const int i = tid * 2 + k * DN_THREADS * 2;
                    hv[k] = i < p.H ? *(const float2*)(hr + i) : make_float2(0.f, 0.f);
                }
#pragma unroll
                for (int k = 0; k < DN_PRE; ++k) {
                    sa += hv[k].x * pa[k].x + hv[k].y * pa[k].y;
                    sb += hv[k].x * pb[k].x + hv[k].y * pb[k].y;
                }
                for (int i = tid * 2 + DN_PRE * DN_THREADS * 2; i < p.H; i += DN_THREADS * 2) {
                    float2 hv2 = *(const float2*)(hr + i);
                    float2 ww = __half22float2(*(const __half2*)(p.ln.w + i));
                    float2 av = __half22float2(*(const __half2*)(wa + i));
                    float2 bv = __half22float2(*(const __half2*)(wb + i));
                    float x0 = hv2.x * ww.x, x1 = hv2.y * ww.y;
                    sa += x0 * av.x + x1 * av.y;
                    sb += x0 * bv.x + x1 * bv.y;
                }
            } else {
                const __half* x = p.xn + (size_t)r * p.ldx;
                float2 xv[DN_PRE];
#pragma unroll
                for (int k = 0; k < DN_PRE; ++k) {
                    const int i = tid * 2 + k * DN_THREADS * 2;
                    xv[k] = i < p.H ? __half22float2(*(const __half2*)(x + i)) : make_float2(0.f, 0.f);
                }
#pragma unroll
                for (int k = 0; k < DN_PRE; ++k) {
                    sa += xv[k].x * pa[k].x + xv[k].y * pa[k].y;
                    sb += xv[k].x * pb[k].x + xv[k].y * pb[k].y;
                }
                for (int i = tid * 2 + DN_PRE * DN_THREADS * 2; i < p.H; i += DN_THREADS * 2) {
                    float2 xv2 = __half22float2(*(const __half2*)(x + i));
                    float2 av = __half22float2(*(const __half2*)(wa + i));
                    float2 bv = __half22float2(*(const __half2*)(wb + i));
                    sa += xv2.x * av.x + xv2.y * av.y;
                    sb += xv2.x * bv.x + xv2.y * bv.y;
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

// ---------------------------------------------------------------------------
// One CTA per value head (all DV columns: DV/32 groups of four warps).  Same arithmetic and the same
// state / conv-history layout as deltanet_step_kernel, laid out for latency: a decode step is a chain of
// short dependent phases, so (1) the sum over the head's columns for the gated RMSNorm goes through shared
// memory instead of a cluster barrier, (2) everything that earlier steps left (state slice, conv history,
// weights of the a/b projections) is in registers before the dependency wait, and (3) all loads that
// depend on this step's in-projection are issued together right after it.
// ---------------------------------------------------------------------------
template <int DK, int DV>
__global__ void __launch_bounds__(DV / 32 * 128) deltanet_head_kernel(const DeltaParams p) {
    constexpr int CB = DV / DN_COLS;
    constexpr int KR = 4;                        // warps sharing one 32-column block: state rows kr, kr + KR, ...
    constexpr int NT = CB * KR * 32;
    constexpr int RPT = DK / KR;                 // state rows per thread
    constexpr int NCHB = 2 * DK + DN_COLS;       // channels per private history copy in memory
    constexpr int NCH = 2 * DK + DV;             // conv channels of the head: q | k | v
    constexpr int PRE = 5;                       // a/b weight pairs per thread kept in registers
    pdl_launch_dependents();
    const int j = blockIdx.x, si = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cb = warp / KR, kr = warp % KR, col = cb * DN_COLS + lane;
    const int kh = j / (p.nv / p.nk);
    const int r0 = p.seq_rows[si], r1 = p.seq_rows[si + 1];
    if (r0 >= r1) return;
    const int seq = p.rows[r0].seq;

    __shared__ float cq[DK], ck[DK], cv[DV];
    __shared__ float red_m[KR][DV], red_q[KR][DV];
    __shared__ float red_ab[NT / 32][2];
    __shared__ float red32[8];
    __shared__ float ss_cb[CB];

    // ---- left by earlier steps: conv history + weights of this thread's channel, state slice, constants
    const bool has_ch = tid < NCH;
    int pcol = 0;
    float h0 = 0.f, h1 = 0.f, h2 = 0.f, w0 = 0.f, w1 = 0.f, w2 = 0.f, w3 = 0.f;
    __half* hist_base = p.conv_state + (((size_t)seq * p.nv + j) * CB) * NCHB * 3;
    __half* my_hist = nullptr;
    if (has_ch) {
        int gch;
        if (tid < DK) { gch = kh * DK + tid; pcol = p.off_q + kh * DK + tid; my_hist = hist_base + (size_t)tid * 3; }
        else if (tid < 2 * DK) { gch = p.nk * DK + kh * DK + (tid - DK); pcol = p.off_k + kh * DK + (tid - DK); my_hist = hist_base + (size_t)tid * 3; }
        else {
            const int v = tid - 2 * DK;
            gch = 2 * p.nk * DK + j * DV + v; pcol = p.off_v + j * DV + v;
            my_hist = hist_base + ((size_t)(v / DN_COLS) * NCHB + 2 * DK + (v % DN_COLS)) * 3;
        }
        h0 = __half2float(my_hist[0]); h1 = __half2float(my_hist[1]); h2 = __half2float(my_hist[2]);
        const __half* w = p.conv_w + (size_t)gch * 4;
        w0 = __half2float(w[0]); w1 = __half2float(w[1]); w2 = __half2float(w[2]); w3 = __half2float(w[3]);
    }
    float S[RPT];
    float* sp = p.state + (((size_t)seq * p.nv + j) * DK) * DV + col;
#pragma unroll
    for (int i = 0; i < RPT; ++i) S[i] = sp[(size_t)(kr + KR * i) * DV];
    const float neg_expA = -__expf(p.A_log[j]);
    const float dtb = __half2float(p.dt_bias[j]);
    const float nw = __half2float(p.norm_w[col]);
    const bool inkernel_ab = p.off_a < 0;
    float2 pa[PRE], pb[PRE];
#pragma unroll
    for (int k = 0; k < PRE; ++k) {
        pa[k] = pb[k] = make_float2(0.f, 0.f);
        const int i = tid * 2 + k * NT * 2;
        if (inkernel_ab && i < p.H) {
            float2 av = __half22float2(*(const __half2*)(p.wa + (size_t)j * p.H + i));
            float2 bv = __half22float2(*(const __half2*)(p.wb + (size_t)j * p.H + i));
            if (p.ln.h) {
                const float2 ww = __half22float2(*(const __half2*)(p.ln.w + i));
                av.x *= ww.x; av.y *= ww.y; bv.x *= ww.x; bv.y *= ww.y;
            }
            pa[k] = av; pb[k] = bv;
        }
    }
    pdl_wait();

    for (int r = r0; r < r1; ++r) {
        const __half* pr = p.proj + (size_t)r * p.ld;
        // ---- every load that depends on this step, issued together
        float2 xin[PRE];
#pragma unroll
        for (int k = 0; k < PRE; ++k) {
            xin[k] = make_float2(0.f, 0.f);
            const int i = tid * 2 + k * NT * 2;
            if (inkernel_ab && i < p.H)
                xin[k] = p.ln.h ? *(const float2*)(p.ln.h + (size_t)r * p.ln.H + i)
                                : __half22float2(*(const __half2*)(p.xn + (size_t)r * p.ldx + i));
        }
        const float xc = has_ch ? __half2float(pr[pcol]) : 0.f;
        const float z = kr == 0 ? __half2float(pr[p.off_z + j * DV + col]) : 0.f;
        float ssp = 0.f, a_dir = 0.f, b_dir = 0.f;
        if (warp == 3) {
            if (inkernel_ab && p.ln.h) for (int i = lane; i < p.ln.np; i += 32) ssp += p.ln.ss[(size_t)r * p.ln.np + i];
            if (!inkernel_ab) { a_dir = __half2float(pr[p.off_a + j]); b_dir = __half2float(pr[p.off_b + j]); }
        }
        // ---- phase A: partial sums of the a/b projections, conv + SiLU of this thread's channel
        if (inkernel_ab) {
            float sa = 0.f, sb = 0.f;
#pragma unroll
            for (int k = 0; k < PRE; ++k) {
                sa += xin[k].x * pa[k].x + xin[k].y * pa[k].y;
                sb += xin[k].x * pb[k].x + xin[k].y * pb[k].y;
            }
            for (int i = tid * 2 + PRE * NT * 2; i < p.H; i += NT * 2) {        // hidden sizes beyond PRE pairs per thread
                float2 xv = p.ln.h ? *(const float2*)(p.ln.h + (size_t)r * p.ln.H + i)
                                   : __half22float2(*(const __half2*)(p.xn + (size_t)r * p.ldx + i));
                float2 av = __half22float2(*(const __half2*)(p.wa + (size_t)j * p.H + i));
                float2 bv = __half22float2(*(const __half2*)(p.wb + (size_t)j * p.H + i));
                if (p.ln.h) {
                    const float2 ww = __half22float2(*(const __half2*)(p.ln.w + i));
                    av.x *= ww.x; av.y *= ww.y; bv.x *= ww.x; bv.y *= ww.y;
                }
                sa += xv.x * av.x + xv.y * av.y;
                sb += xv.x * bv.x + xv.y * bv.y;
            }
            sa = warp_sum(sa);
            sb = warp_sum(sb);
            if (lane == 0) { red_ab[warp][0] = sa; red_ab[warp][1] = sb; }
        }
        if (has_ch) {
            float o = silu_f(h0 * w0 + h1 * w1 + h2 * w2 + xc * w3);
            h0 = h1; h1 = h2; h2 = xc;
            if (tid < DK) cq[tid] = o; else if (tid < 2 * DK) ck[tid - DK] = o; else cv[tid - 2 * DK] = o;
        }
        __syncthreads();
        // ---- phase B: warps 0..2 the q/k norms and q.k, warp 3 the a/b inputs
        if (warp < 3) {
            float s = 0.f;
            for (int i = lane; i < DK; i += 32) {
                float a = (warp == 1) ? ck[i] : cq[i], b = (warp == 0) ? cq[i] : ck[i];
                s += a * b;                      // warp 0: q.q  warp 1: k.k  warp 2: q.k
            }
            s = warp_sum(s);
            if (lane == 0) red32[warp] = s;
        } else if (warp == 3) {
            float a_in = a_dir, b_in = b_dir;
            if (inkernel_ab) {
                float inv = 1.f;
                if (p.ln.h) inv = rsqrtf(warp_sum(ssp) / (float)p.ln.H + p.ln.eps);
                float ta = 0.f, tb = 0.f;
                for (int w = lane; w < NT / 32; w += 32) { ta += red_ab[w][0]; tb += red_ab[w][1]; }
                ta = warp_sum(ta); tb = warp_sum(tb);
                // the unfused path rounds the projection output to fp16: keep that rounding
                a_in = __half2float(__float2half(ta * inv));
                b_in = __half2float(__float2half(tb * inv));
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
            mp = fmaf(S[i], ck[kr + KR * i], mp);
            qp = fmaf(S[i], cq[kr + KR * i], qp);
        }
        red_m[kr][col] = mp * invk;
        red_q[kr][col] = qp * invq;
        __syncthreads();
        float mm = 0.f, sq = 0.f;
#pragma unroll
        for (int w = 0; w < KR; ++w) { mm += red_m[w][col]; sq += red_q[w][col]; }
        const float delta = (cv[col] - decay * mm) * beta;
        const float y = decay * sq + delta * kq;
#pragma unroll
        for (int i = 0; i < RPT; ++i) S[i] = decay * S[i] + ck[kr + KR * i] * invk * delta;
        // ---- gated RMSNorm over the head's DV outputs
        const float ss = warp_sum(y * y);
        if (kr == 0 && lane == 0) ss_cb[cb] = ss;
        __syncthreads();
        if (kr == 0) {
            float tot = 0.f;
#pragma unroll
            for (int c = 0; c < CB; ++c) tot += ss_cb[c];
            float o = y * rsqrtf(tot / (float)DV + p.eps) * nw * silu_f(z);
            p.out[(size_t)r * p.ldo + j * DV + col] = __float2half(o);
        }
        __syncthreads();                         // this row's shared-memory reads before the next row's writes
    }
    if (!p.commit) return;
#pragma unroll
    for (int i = 0; i < RPT; ++i) sp[(size_t)(kr + KR * i) * DV] = S[i];
    if (has_ch) {
        const __half a0 = __float2half(h0), a1 = __float2half(h1), a2 = __float2half(h2);
        if (tid < 2 * DK) {
            // q / k history: every column block keeps its own copy (the chunked scan and the verify kernels read them)
#pragma unroll
            for (int c = 0; c < CB; ++c) {
                __half* d = hist_base + ((size_t)c * NCHB + tid) * 3;
                d[0] = a0; d[1] = a1; d[2] = a2;
            }
        } else {
            my_hist[0] = a0; my_hist[1] = a1; my_hist[2] = a2;
        }
    }
}

template <int DK, int DV>
static int launch_delta_head(const DeltaParams* p, cudaStream_t s) {
    return launch_pdl(deltanet_head_kernel<DK, DV>, dim3(p->nv, p->n_seqs), dim3(DV / 32 * 128), 0, s, *p);
}

template <int DK, int DV>
static int launch_delta(const DeltaParams* p, cudaStream_t s) {
    constexpr int CB = DV / DN_COLS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(CB, p->nv, p->n_seqs);
    cfg.blockDim = dim3(DN_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CB;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: the CTAs become resident, load their state slice, conv history and
    // weights while the in-projection is still finishing, and wait (griddepcontrol.wait) only then
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, deltanet_step_kernel<DK, DV>, *p);
}

B2_API int b2_deltanet_step(const DeltaParams* p, int dk, int dv, cudaStream_t s) {
    if (p->nv % p->nk) return cudaErrorInvalidValue;
    // one CTA per head (deltanet_head_kernel) unless B200GRAD_DELTANET_CLUSTER selects the cluster form
    static const bool cluster_form = getenv("B200GRAD_DELTANET_CLUSTER") != nullptr;
    if (!cluster_form) {
        if (dk == 128 && dv == 128) return launch_delta_head<128, 128>(p, s);
        if (dk == 64 && dv == 64) return launch_delta_head<64, 64>(p, s);
    }
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
#define DC_C 32                  // rows per chunk: small enough that two CTAs share an SM and overlap their phases
#define DC_LDK(DK) ((DK) + 4)    // padded row stride of the q/k tiles (conflict-free fragment loads)
#define DC_LDA (DC_C + 4)
#define DC_LDU (DN_COLS + 8)     // row stride of U and of the state copy (they are B operands)

// The matrix products of a chunk run on the tensor cores as TF32 (fp32 storage, 10-bit
// mantissa: the precision of the fp16 activations the inputs come from), accumulating in fp32.
__device__ __forceinline__ float tf32r(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], float a0, float a1, float a2, float a3, float b0, float b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(__float_as_uint(a0)), "r"(__float_as_uint(a1)), "r"(__float_as_uint(a2)), "r"(__float_as_uint(a3)),
                   "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// Four 8x4 fp32 tiles in one instruction: lane l supplies the address of row (l & 7) of tile l >> 3
// (16 bytes = 4 floats per row); afterwards every lane holds element (lane >> 2, lane & 3) of each
// tile, which is exactly the TF32 fragment layout of mma.m16n8k8.
__device__ __forceinline__ void ldsm4(float (&r)[4], const float* row_ptr) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(row_ptr);
    uint32_t x0, x1, x2, x3;
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(a));
    r[0] = __uint_as_float(x0); r[1] = __uint_as_float(x1); r[2] = __uint_as_float(x2); r[3] = __uint_as_float(x3);
}
__device__ __forceinline__ void ldsm2(float (&r)[2], const float* row_ptr) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(row_ptr);
    uint32_t x0, x1;
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(x0), "=r"(x1) : "r"(a));
    r[0] = __uint_as_float(x0); r[1] = __uint_as_float(x1);
}
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.f + __expf(-x)); }

template <int DK, int DV>
__global__ void __launch_bounds__(DN_THREADS, 2) deltanet_chunk_kernel(const DeltaParams p, const __half* __restrict__ ab, int ld_ab,
                                                                      const __half* __restrict__ qk_pre, int ld_qk,
                                                                      const float* __restrict__ tw_pre, int n_chunks) {
    constexpr int CB = DV / DN_COLS;
    constexpr int MT = DK / 16;               // 16-row tiles of the state slice, one or two per warp
    constexpr int SPW = (MT + 7) / 8;         // state m-tiles per warp
    constexpr int NCH = 2 * DK + DN_COLS;
    constexpr int LDK = DC_LDK(DK);
    static_assert(DK % 16 == 0 && MT <= 16, "state tiling");
    cg::cluster_group cluster = cg::this_cluster();
    pdl_launch_dependents();
    const int cb = blockIdx.x, j = blockIdx.y, si = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, kr = tid >> 5, vcol = lane;
    const int g = lane >> 2, t = lane & 3;    // fragment coordinates
    const int kh = j / (p.nv / p.nk);
    const int r0 = p.seq_rows[si], r1 = p.seq_rows[si + 1];
    if (r0 >= r1) return;
    const int seq = p.rows[r0].seq;

    extern __shared__ __align__(16) float dsm[];
    float* Qs = dsm;                          // [C][LDK]
    float* Ks = Qs + DC_C * LDK;              // [C][LDK]
    float* Us = Ks + DC_C * LDK;              // [C][LDU]  v -> b -> u (in place)
    float* QSs = Us + DC_C * DC_LDU;          // [C][32]   exp(G) Q S0
    float* Ys = QSs + DC_C * DN_COLS;         // [C][32]
    float* As0 = Ys + DC_C * DN_COLS;         // [2][2][C][LDA]: (A or T, W) of this chunk and, with the pre-pass, of the next
    float* S0t = As0 + 4 * DC_C * DC_LDA;     // [32][LDK]  transposed copy of the state slice (a B operand)
    float* hist = S0t + DN_COLS * LDK;        // [NCH][3]
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
        for (int q = 0; q < 3; ++q) hist[c * 3 + q] = __half2float(my_hist[c * 3 + q]);
        const __half* w = p.conv_w + (size_t)chan(c) * 4;
#pragma unroll
        for (int q = 0; q < 4; ++q) cw[c * 4 + q] = __half2float(w[q]);
    }
    // The state slice [DK x 32] lives in registers as accumulator fragments: warp w owns the
    // 16-row tiles w (and w + 8), each as four 16x8 tiles: S[m][n][0..3] = rows g / g+8, cols 2t / 2t+1.
    float S[SPW][4][4];
    float* sp = p.state + (((size_t)seq * p.nv + j) * DK) * DV + cb * DN_COLS;
#pragma unroll
    for (int m = 0; m < SPW; ++m) {
        const int mt = kr + 8 * m;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            if (mt < MT) {
                const float2 lo = *(const float2*)(sp + (size_t)(16 * mt + g) * DV + 8 * n + 2 * t);
                const float2 hi = *(const float2*)(sp + (size_t)(16 * mt + g + 8) * DV + 8 * n + 2 * t);
                S[m][n][0] = lo.x; S[m][n][1] = lo.y; S[m][n][2] = hi.x; S[m][n][3] = hi.y;
            } else {
                S[m][n][0] = S[m][n][1] = S[m][n][2] = S[m][n][3] = 0.f;
            }
        }
    }
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
            if (qk_pre && c < 2 * DK) {
                // q / k columns: convolved, normalised (q also scaled) rows from the pre-pass; no history rows
                if (ri >= rb_ && ri < r1)
                    cp_async16(dst, qk_pre + (size_t)(ri - r0) * ld_qk + (c < DK ? kh * DK + c : p.nk * DK + kh * DK + (c - DK)));
                else
                    *(uint4*)dst = make_uint4(0u, 0u, 0u, 0u);
            } else if (ri >= r0 && ri < r1) {
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
    // T = (I + A)^-1 and W of a chunk from the pre-pass: 32 x 32 floats each, into the chunk's pair of buffers
    auto stage_tw = [&](int ci) {
        if (!tw_pre) return;
        float* dstb = As0 + (ci & 1) * 2 * DC_C * DC_LDA;
        const float* src = tw_pre + ((size_t)j * n_chunks + ci) * 2 * DC_C * DC_C;
        for (int idx = tid; idx < 2 * DC_C * (DC_C / 4); idx += DN_THREADS) {
            const int mat = idx / (DC_C * (DC_C / 4)), rem = idx % (DC_C * (DC_C / 4));
            const int row = rem / (DC_C / 4), pc = rem % (DC_C / 4);
            cp_async16(dstb + mat * DC_C * DC_LDA + row * DC_LDA + pc * 4, src + mat * DC_C * DC_C + row * DC_C + pc * 4);
        }
    };
    stage_tw(0);
    stage_raw(r0);
    // the gate inputs of a chunk are fetched one chunk ahead (a global round trip off the critical path)
    float a_pre = 0.f, b_pre = 0.f;
    auto fetch_gates = [&](int rb_) {
        a_pre = b_pre = 0.f;
        if (tid < DC_C && rb_ + tid < r1) {
            const __half* abr = ab + (size_t)(rb_ + tid) * ld_ab;
            a_pre = __half2float(abr[j]); b_pre = __half2float(abr[p.nv + j]);
        }
    };
    fetch_gates(r0);

    int chunk_idx = 0;
    for (int rb = r0; rb < r1; rb += DC_C, ++chunk_idx) {
        const int Ce = min(DC_C, r1 - rb);
        const int slot = chunk_idx & 1;
        // ---- P1: causal conv + SiLU from the raw tile staged in shared memory by cp.async (the
        // copy for this chunk was issued while the previous chunk was being processed)
        cp_async_wait<0>();
        __syncthreads();
        // two adjacent channels per item (one 4-byte shared-memory load serves both), 8 rows per item
        for (int item = tid; item < (NCH / 2) * (DC_C / 8); item += DN_THREADS) {
            const int c = 2 * (item % (NCH / 2)), i0 = (item / (NCH / 2)) * 8;
            const float4 wa4 = *(const float4*)&cw[c * 4], wb4 = *(const float4*)&cw[c * 4 + 4];
            float* dst = (c < DK) ? Qs + c : (c < 2 * DK) ? Ks + (c - DK) : Us + (c - 2 * DK);
            const int ldd = (c < 2 * DK) ? LDK : DC_LDU;
            if (qk_pre && c < 2 * DK) {
                // already convolved and normalised by the pre-pass (fp16 holds exactly the ten mantissa bits the
                // TF32 products use): widen and store
#pragma unroll
                for (int i = i0; i < i0 + 8; ++i)
                    *(float2*)&dst[i * ldd] = __half22float2(*(const __half2*)&Xr[(i + 3) * NCH + c]);
                continue;
            }
            float2 x0 = __half22float2(*(const __half2*)&Xr[(i0 + 0) * NCH + c]);
            float2 x1 = __half22float2(*(const __half2*)&Xr[(i0 + 1) * NCH + c]);
            float2 x2 = __half22float2(*(const __half2*)&Xr[(i0 + 2) * NCH + c]);
#pragma unroll
            for (int i = i0; i < i0 + 8; ++i) {
                const float2 x3 = __half22float2(*(const __half2*)&Xr[(i + 3) * NCH + c]);
                const float a0 = x0.x * wa4.x + x1.x * wa4.y + x2.x * wa4.z + x3.x * wa4.w;
                const float a1 = x0.y * wb4.x + x1.y * wb4.y + x2.y * wb4.z + x3.y * wb4.w;
                *(float2*)&dst[i * ldd] = (i < Ce) ? make_float2(silu_fast(a0), silu_fast(a1)) : make_float2(0.f, 0.f);
                x0 = x1; x1 = x2; x2 = x3;
            }
        }
        if (tid < DC_C) {
            float gl = 0.f, beta = 0.f;
            if (tid < Ce) {
                const float a_in = a_pre, b_in = b_pre;
                float sp_ = a_in + dtb;
                gl = fmaxf(neg_expA * (sp_ > 20.f ? sp_ : log1pf(__expf(sp_))), -20.f);
                beta = sigmoid_f(b_in);
            }
            gs[tid] = gl;
            bs[tid] = beta;
            cl_ss[slot * DC_C + tid] = 0.f;
        }
        __syncthreads();
        if (rb + DC_C < r1) { stage_tw(chunk_idx + 1); stage_raw(rb + DC_C); }          // fly while this chunk is processed
        float* As = As0 + (tw_pre ? (chunk_idx & 1) * 2 * DC_C * DC_LDA : 0);
        float* Ws = As + DC_C * DC_LDA;
        fetch_gates(rb + DC_C);
        // output gates of this chunk, needed only at its end
        float zf[DC_C / 8];
#pragma unroll
        for (int u = 0; u < DC_C / 8; ++u) {
            const int i = kr + 8 * u;
            zf[u] = (i < Ce) ? __half2float(p.proj[(size_t)(rb + i) * p.ld + p.off_z + j * DV + cb * DN_COLS + vcol]) : 0.f;
        }
        // ---- P2: L2-normalise q and k rows (stored rounded to TF32), running log-decay, state copy
        if (kr == 0) {
            // inclusive scan of the log-decays: DC_C / 32 per lane
            static_assert(DC_C == 32 || DC_C == 64, "chunk size");
            float a = gs[lane], b = DC_C > 32 ? gs[lane + DC_C - 32] : 0.f;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float ua = __shfl_up_sync(0xffffffffu, a, o), ub = __shfl_up_sync(0xffffffffu, b, o);
                if (lane >= o) { a += ua; b += ub; }
            }
            const float tot = __shfl_sync(0xffffffffu, a, 31);
            Gs[lane] = a;
            if (DC_C > 32) Gs[lane + DC_C - 32] = b + tot;
        }
#pragma unroll 1
        for (int ub = 0; ub < (qk_pre ? 0 : DC_C / 8); ub += 4) {
            // four rows at a time: their loads and the eight reductions overlap
            constexpr int PL = DK / 32;
            float qv[4][PL], kv[4][PL], qq[4], kk[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int i = kr + 8 * (ub + r);
                qq[r] = kk[r] = 0.f;
#pragma unroll
                for (int m = 0; m < PL; ++m) {
                    qv[r][m] = Qs[i * LDK + lane + 32 * m]; kv[r][m] = Ks[i * LDK + lane + 32 * m];
                    qq[r] += qv[r][m] * qv[r][m]; kk[r] += kv[r][m] * kv[r][m];
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    qq[r] += __shfl_xor_sync(0xffffffffu, qq[r], o);
                    kk[r] += __shfl_xor_sync(0xffffffffu, kk[r], o);
                }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int i = kr + 8 * (ub + r);
                const float iq = rsqrtf(qq[r] + 1e-6f) * qscale, ik = rsqrtf(kk[r] + 1e-6f);
#pragma unroll
                for (int m = 0; m < PL; ++m) {
                    Qs[i * LDK + lane + 32 * m] = tf32r(qv[r][m] * iq);
                    Ks[i * LDK + lane + 32 * m] = tf32r(kv[r][m] * ik);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < SPW; ++m) {
            const int mt = kr + 8 * m;
            if (mt < MT) {
#pragma unroll
                for (int n = 0; n < 4; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        S0t[(8 * n + 2 * t + (e & 1)) * LDK + 16 * mt + g + (e >> 1) * 8] = tf32r(S[m][n][e]);
            }
        }
        __syncthreads();
        // ---- P3: A = beta decay (K K^T) below the diagonal, W = decay (Q K^T) on and below it, in
        // 16x8 tiles of the lower triangle dealt round-robin to the warps.  Fragments come from
        // ldmatrix: one instruction per operand and k-step.
        constexpr int MB = DC_C / 16;                 // 16-row blocks of a chunk
        constexpr int NTW = (MB * 4) / 8;             // 8-column tiles of U / Y per warp in P4 and P6 (1 or 2)
        const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 4;       // A operand addressing
        const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 4;       // B operand, two 8-column tiles
        {
            for (int tile = kr; tile < (tw_pre ? 0 : MB * (MB + 1)); tile += 8) {
                int mi = 0, ni = tile;                 // row block mi holds tiles ni = 0 .. 2 mi + 1
                while (ni >= 2 * mi + 2) { ni -= 2 * mi + 2; ++mi; }
                float kk[4] = {0.f, 0.f, 0.f, 0.f}, qk[4] = {0.f, 0.f, 0.f, 0.f};
                const float* ka = Ks + (16 * mi + a_row) * LDK + a_col;
                const float* qa = Qs + (16 * mi + a_row) * LDK + a_col;
                const float* kb = Ks + (8 * ni + (lane & 7)) * LDK + ((lane >> 3) & 1) * 4;   // x2: lanes 0-15 give the rows
#pragma unroll 4
                for (int k0 = 0; k0 < DK; k0 += 8) {
                    float fa[4], fq[4], fb[2];
                    ldsm4(fa, ka + k0); ldsm4(fq, qa + k0); ldsm2(fb, kb + k0);
                    mma_tf32(kk, fa[0], fa[1], fa[2], fa[3], fb[0], fb[1]);
                    mma_tf32(qk, fq[0], fq[1], fq[2], fq[3], fb[0], fb[1]);
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = 16 * mi + g + (e >> 1) * 8, jj = 8 * ni + 2 * t + (e & 1);
                    const float dec = (jj <= i) ? __expf(Gs[i] - Gs[jj]) : 0.f;
                    As[i * DC_LDA + jj] = (jj < i) ? bs[i] * dec * kk[e] : 0.f;
                    Ws[i * DC_LDA + jj] = tf32r(dec * qk[e]);
                }
            }
            // ---- P4: K S0 and Q S0; b = beta (v - exp(G) K S0) in place of v.  Warp w: row block
            // w % MB, column tiles NTW (w / MB) ...
            const int mi = kr % MB, nb = (kr / MB) * NTW;
            float ak[NTW][4], aq[NTW][4];
#pragma unroll
            for (int n = 0; n < NTW; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) ak[n][e] = aq[n][e] = 0.f;
            const float* ka = Ks + (16 * mi + a_row) * LDK + a_col;
            const float* qa = Qs + (16 * mi + a_row) * LDK + a_col;
            const float* sb4 = S0t + (8 * nb + b_row) * LDK + b_col;
            const float* sb2 = S0t + (8 * nb + (lane & 7)) * LDK + ((lane >> 3) & 1) * 4;
#pragma unroll 4
            for (int k0 = 0; k0 < DK; k0 += 8) {
                float fa[4], fq[4], fb[4];
                ldsm4(fa, ka + k0); ldsm4(fq, qa + k0);
                if constexpr (NTW == 2) {
                    ldsm4(fb, sb4 + k0);
                } else {
                    float f2[2];
                    ldsm2(f2, sb2 + k0);
                    fb[0] = f2[0]; fb[1] = f2[1]; fb[2] = fb[3] = 0.f;
                }
#pragma unroll
                for (int n = 0; n < NTW; ++n) {
                    mma_tf32(ak[n], fa[0], fa[1], fa[2], fa[3], fb[2 * n], fb[2 * n + 1]);
                    mma_tf32(aq[n], fq[0], fq[1], fq[2], fq[3], fb[2 * n], fb[2 * n + 1]);
                }
            }
#pragma unroll
            for (int n = 0; n < NTW; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = 16 * mi + g + (e >> 1) * 8, col = 8 * (nb + n) + 2 * t + (e & 1);
                    const float eg = __expf(Gs[i]);
                    Us[i * DC_LDU + col] = bs[i] * (Us[i * DC_LDU + col] - eg * ak[n][e]);
                    QSs[i * DN_COLS + col] = eg * aq[n][e];
                }
        }
        __syncthreads();
        // ---- P5: (I + A) U = B by forward substitution, 8 rows per block: every warp first removes
        // the contribution of all earlier blocks from its row, then warp 0 solves the 8x8 triangle
        // with one column per lane in registers
        if (tw_pre) {
            // U = T B with T = (I + A)^-1 from the pre-pass: one 16x8 tile per warp, split-TF32 operands
            // (hi + lo parts) so that the product keeps fp32 accuracy like the substitution it replaces
            const int mi5 = kr % MB, nb5 = (kr / MB) * NTW;
            float u[NTW][4];
#pragma unroll
            for (int n = 0; n < NTW; ++n) u[n][0] = u[n][1] = u[n][2] = u[n][3] = 0.f;
            const float* ta = As + (16 * mi5 + a_row) * DC_LDA + a_col;
            for (int k0 = 0; k0 < 16 * (mi5 + 1); k0 += 8) {
                float fa[4], hi[4], lo[4];
                ldsm4(fa, ta + k0);
#pragma unroll
                for (int e = 0; e < 4; ++e) { hi[e] = tf32r(fa[e]); lo[e] = tf32r(fa[e] - hi[e]); }
#pragma unroll
                for (int n = 0; n < NTW; ++n) {
                    const float b0 = Us[(k0 + t) * DC_LDU + 8 * (nb5 + n) + g], b1 = Us[(k0 + t + 4) * DC_LDU + 8 * (nb5 + n) + g];
                    const float b0h = tf32r(b0), b1h = tf32r(b1);
                    mma_tf32(u[n], lo[0], lo[1], lo[2], lo[3], b0h, b1h);
                    mma_tf32(u[n], hi[0], hi[1], hi[2], hi[3], tf32r(b0 - b0h), tf32r(b1 - b1h));
                    mma_tf32(u[n], hi[0], hi[1], hi[2], hi[3], b0h, b1h);
                }
            }
            __syncthreads();                               // every warp has read B before anyone overwrites it
#pragma unroll
            for (int n = 0; n < NTW; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    Us[(16 * mi5 + g + (e >> 1) * 8) * DC_LDU + 8 * (nb5 + n) + 2 * t + (e & 1)] = u[n][e];
            __syncthreads();
        } else
        for (int blk = 0; blk < DC_C / 8; ++blk) {
            const int i = 8 * blk + kr;
            float acc = Us[i * DC_LDU + vcol];
            for (int j0 = 0; j0 < 8 * blk; j0 += 8) {
                float av[8], uv[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) { av[q] = As[i * DC_LDA + j0 + q]; uv[q] = Us[(j0 + q) * DC_LDU + vcol]; }
#pragma unroll
                for (int q = 0; q < 8; ++q) acc = fmaf(-av[q], uv[q], acc);
            }
            Us[i * DC_LDU + vcol] = acc;
            __syncthreads();
            if (kr == 0) {
                float u[8];
#pragma unroll
                for (int a = 0; a < 8; ++a) u[a] = Us[(8 * blk + a) * DC_LDU + vcol];
#pragma unroll
                for (int a = 1; a < 8; ++a)
#pragma unroll
                    for (int b = 0; b < 8; ++b)
                        if (b < a) u[a] = fmaf(-As[(8 * blk + a) * DC_LDA + 8 * blk + b], u[b], u[a]);
#pragma unroll
                for (int a = 1; a < 8; ++a) Us[(8 * blk + a) * DC_LDU + vcol] = u[a];
            }
            __syncthreads();
        }
        // ---- P6: Y = exp(G) Q S0 + W U (W is zero above the diagonal), sum of squares per row
        {
            const int mi = kr % MB, nb = (kr / MB) * NTW;
            float y[NTW][4];
#pragma unroll
            for (int n = 0; n < NTW; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    y[n][e] = QSs[(16 * mi + g + (e >> 1) * 8) * DN_COLS + 8 * (nb + n) + 2 * t + (e & 1)];
            const float* wa = Ws + (16 * mi + a_row) * DC_LDA + a_col;
            for (int k0 = 0; k0 < 16 * (mi + 1); k0 += 8) {
                float fa[4];
                ldsm4(fa, wa + k0);
#pragma unroll
                for (int n = 0; n < NTW; ++n)
                    mma_tf32(y[n], fa[0], fa[1], fa[2], fa[3], tf32r(Us[(k0 + t) * DC_LDU + 8 * (nb + n) + g]),
                             tf32r(Us[(k0 + t + 4) * DC_LDU + 8 * (nb + n) + g]));
            }
            float s_lo = 0.f, s_hi = 0.f;
#pragma unroll
            for (int n = 0; n < NTW; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    Ys[(16 * mi + g + (e >> 1) * 8) * DN_COLS + 8 * (nb + n) + 2 * t + (e & 1)] = y[n][e];
                    if (e < 2) s_lo += y[n][e] * y[n][e]; else s_hi += y[n][e] * y[n][e];
                }
            s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 1); s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 2);
            s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 1); s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 2);
            if (t == 0) {
                atomicAdd(&cl_ss[slot * DC_C + 16 * mi + g], s_lo);
                atomicAdd(&cl_ss[slot * DC_C + 16 * mi + g + 8], s_hi);
            }
        }
        // ---- P7: S' = exp(G_C) S0 + K^T (exp(G_C - G) U), accumulated into the register fragments
        {
            const float gC = Gs[DC_C - 1];
            const float egC = __expf(gC);
#pragma unroll
            for (int m = 0; m < SPW; ++m)
#pragma unroll
                for (int n = 0; n < 4; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) S[m][n][e] *= egC;
            for (int k0 = 0; k0 < DC_C; k0 += 8) {
                const float tl0 = __expf(gC - Gs[k0 + t]), tl1 = __expf(gC - Gs[k0 + t + 4]);
                float b0[4], b1[4];
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    b0[n] = tf32r(Us[(k0 + t) * DC_LDU + 8 * n + g] * tl0);
                    b1[n] = tf32r(Us[(k0 + t + 4) * DC_LDU + 8 * n + g] * tl1);
                }
#pragma unroll
                for (int m = 0; m < SPW; ++m) {
                    const int mt = kr + 8 * m;
                    if (mt < MT) {
                        // A = K^T: element (dk row, chunk row) = Ks[chunk row][dk row]
                        const float* kt = Ks + (k0 + t) * LDK + 16 * mt + g;
                        const float a0 = kt[0], a1 = kt[8], a2 = kt[4 * LDK], a3 = kt[4 * LDK + 8];
#pragma unroll
                        for (int n = 0; n < 4; ++n) mma_tf32(S[m][n], a0, a1, a2, a3, b0[n], b1[n]);
                    }
                }
            }
        }
        cluster.sync();
        // ---- gated RMSNorm across the head's column blocks, output.  The warp's DC_C/8 rows x CB
        // peers are read from distributed shared memory by that many lanes at once, and the gate values are
        // loaded before anything is stored.
        {
            float v = 0.f;
            if (lane < (DC_C / 8) * CB) v = cluster.map_shared_rank(cl_ss, lane % CB)[slot * DC_C + kr + 8 * (lane / CB)];
#pragma unroll
            for (int o = CB / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
#pragma unroll
            for (int u = 0; u < DC_C / 8; ++u) {
                const int i = kr + 8 * u;
                const float tot = __shfl_sync(0xffffffffu, v, u * CB);
                if (i < Ce) {
                    const float o = Ys[i * DN_COLS + vcol] * rsqrtf(tot / (float)DV + p.eps) * nw * silu_fast(zf[u]);
                    p.out[(size_t)(rb + i) * p.ldo + j * DV + cb * DN_COLS + vcol] = __float2half(o);
                }
            }
        }
        __syncthreads();
    }
    cluster.sync();
    if (!p.commit) return;
#pragma unroll
    for (int m = 0; m < SPW; ++m) {
        const int mt = kr + 8 * m;
        if (mt < MT) {
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                *(float2*)(sp + (size_t)(16 * mt + g) * DV + 8 * n + 2 * t) = make_float2(S[m][n][0], S[m][n][1]);
                *(float2*)(sp + (size_t)(16 * mt + g + 8) * DV + 8 * n + 2 * t) = make_float2(S[m][n][2], S[m][n][3]);
            }
        }
    }
    // last three raw conv inputs (older history shifts in when the sequence was shorter than 3 rows)
    for (int c = tid; c < NCH; c += DN_THREADS) {
        const int col = proj_col(c);
#pragma unroll
        for (int q = 0; q < 3; ++q) {
            const int ri = r1 - 3 + q;
            float x = (ri >= r0) ? __half2float(p.proj[(size_t)ri * p.ld + col]) : hist[c * 3 + (ri - r0 + 3)];
            my_hist[c * 3 + q] = __float2half(x);
        }
    }
}

// ---------------------------------------------------------------------------
// Pre-pass of the chunked scan: causal conv + SiLU + L2 norm of the q and k channels of every row, once
// per key head and fully parallel over the rows (the scan kernel would otherwise redo it in each of the
// dv/32 column CTAs of each of the nv/nk value heads that share a key head, on its sequential path).
// Output fp16 [rows][2 * nk * DK]: q (scaled by 1/sqrt(DK)) | k.  grid = (row blocks of QP_ROWS, key heads),
// 2 * DK threads: thread c owns one channel for QP_ROWS rows.
// ---------------------------------------------------------------------------
#define QP_ROWS 16
template <int DK>
__global__ void __launch_bounds__(2 * DK) deltanet_qk_prep_kernel(const DeltaParams p, __half* __restrict__ qk_pre, int ld_qk,
                                                                  int cb_copies, int nch) {
    const int kh = blockIdx.y, c = threadIdx.x, lane = c & 31, warp = c >> 5;
    const int r0 = p.seq_rows[0], r1 = p.seq_rows[1];
    const int rb = r0 + blockIdx.x * QP_ROWS;
    if (rb >= r1) return;
    const int seq = p.rows[r0].seq;
    const bool is_q = c < DK;
    const int gch = is_q ? kh * DK + c : p.nk * DK + kh * DK + (c - DK);
    const int col = is_q ? p.off_q + kh * DK + c : p.off_k + kh * DK + (c - DK);
    const __half* w = p.conv_w + (size_t)gch * 4;
    const float w0 = __half2float(w[0]), w1 = __half2float(w[1]), w2 = __half2float(w[2]), w3 = __half2float(w[3]);
    // rows before the sequence start come from the saved history of the first value head of this key head
    const __half* hist = p.conv_state + ((((size_t)seq * p.nv + kh * (p.nv / p.nk)) * cb_copies) * nch + c) * 3;
    auto input = [&](int ri) -> float {
        if (ri >= r1) return 0.f;
        return ri >= r0 ? __half2float(p.proj[(size_t)ri * p.ld + col]) : __half2float(hist[ri - r0 + 3]);
    };
    float x[QP_ROWS + 3];
#pragma unroll
    for (int i = 0; i < QP_ROWS + 3; ++i) x[i] = input(rb - 3 + i);
    __shared__ float part[2 * DK / 32][QP_ROWS];
    float y[QP_ROWS];
#pragma unroll
    for (int i = 0; i < QP_ROWS; ++i) {
        y[i] = silu_fast(x[i] * w0 + x[i + 1] * w1 + x[i + 2] * w2 + x[i + 3] * w3);
        const float ss = warp_sum(y[i] * y[i]);
        if (lane == 0) part[warp][i] = ss;
    }
    __syncthreads();
    const int w_lo = is_q ? 0 : DK / 32;
    const float qscale = is_q ? rsqrtf((float)DK) : 1.f;
#pragma unroll
    for (int i = 0; i < QP_ROWS; ++i) {
        if (rb + i >= r1) break;
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < DK / 32; ++k) ss += part[w_lo + k][i];
        qk_pre[(size_t)(rb - r0 + i) * ld_qk + (is_q ? kh * DK + c : p.nk * DK + kh * DK + (c - DK))] =
            __float2half_rn(y[i] * rsqrtf(ss + 1e-6f) * qscale);
    }
}

// ---------------------------------------------------------------------------
// Second pre-pass of the chunked scan: everything of a chunk that does not depend on the state, for every
// (value head, chunk) in parallel: the gates, A = beta decay (K K^T) below the diagonal, W = decay (Q K^T) on
// and below it, and T = (I + A)^-1 (forward substitution on the 32 x 32 unit triangle, one column per lane).
// The scan then replaces its per-chunk products and its sequential triangular solve by loads and U = T B.
// Output fp32 [nv][n_chunks][T | W][32][32].  grid = (chunks, value heads), 256 threads.
// ---------------------------------------------------------------------------
template <int DK>
__global__ void __launch_bounds__(DN_THREADS) deltanet_tw_prep_kernel(const DeltaParams p, const __half* __restrict__ ab, int ld_ab,
                                                                      const __half* __restrict__ qk_pre, int ld_qk,
                                                                      float* __restrict__ tw, int n_chunks) {
    static_assert(DC_C == 32, "one lane per column of the triangle");
    constexpr int LDK = DC_LDK(DK);
    constexpr int MB = DC_C / 16;
    extern __shared__ __align__(16) float psm[];
    float* Qs = psm;                          // [C][LDK]
    float* Ks = Qs + DC_C * LDK;
    float* As = Ks + DC_C * LDK;              // [C][LDA]
    float* Ws = As + DC_C * DC_LDA;
    float* Ts = Ws + DC_C * DC_LDA;
    float* Gs = Ts + DC_C * DC_LDA;           // [C]
    float* bs = Gs + DC_C;
    float* gs = bs + DC_C;
    const int ci = blockIdx.x, j = blockIdx.y, kh = j / (p.nv / p.nk);
    const int tid = threadIdx.x, lane = tid & 31, kr = tid >> 5, g = lane >> 2, t = lane & 3;
    const int r0 = p.seq_rows[0], r1 = p.seq_rows[1];
    const int rb = r0 + ci * DC_C;
    if (rb >= r1) return;
    const int Ce = min(DC_C, r1 - rb);
    for (int idx = tid; idx < DC_C * (DK / 8) * 2; idx += DN_THREADS) {
        const int which = idx / (DC_C * (DK / 8)), rem = idx % (DC_C * (DK / 8));
        const int row = rem / (DK / 8), c = (rem % (DK / 8)) * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < Ce) v = *(const uint4*)(qk_pre + (size_t)(rb - r0 + row) * ld_qk + (which ? p.nk * DK : 0) + kh * DK + c);
        const __half2* h2 = (const __half2*)&v;
        float* dst = (which ? Ks : Qs) + row * LDK + c;
#pragma unroll
        for (int q = 0; q < 4; ++q) { const float2 f = __half22float2(h2[q]); dst[2 * q] = f.x; dst[2 * q + 1] = f.y; }
    }
    if (tid < DC_C) {
        float gl = 0.f, beta = 0.f;
        if (tid < Ce) {
            const __half* abr = ab + (size_t)(rb + tid) * ld_ab;
            const float sp_ = __half2float(abr[j]) + __half2float(p.dt_bias[j]);
            gl = fmaxf(-__expf(p.A_log[j]) * (sp_ > 20.f ? sp_ : log1pf(__expf(sp_))), -20.f);
            beta = sigmoid_f(__half2float(abr[p.nv + j]));
        }
        gs[tid] = gl;
        bs[tid] = beta;
    }
    __syncthreads();
    if (kr == 0) {
        float a = gs[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float ua = __shfl_up_sync(0xffffffffu, a, o);
            if (lane >= o) a += ua;
        }
        Gs[lane] = a;
    }
    __syncthreads();
    {
        const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 4;
        for (int tile = kr; tile < MB * (MB + 1); tile += 8) {
            int mi = 0, ni = tile;
            while (ni >= 2 * mi + 2) { ni -= 2 * mi + 2; ++mi; }
            float kk[4] = {0.f, 0.f, 0.f, 0.f}, qk[4] = {0.f, 0.f, 0.f, 0.f};
            const float* ka = Ks + (16 * mi + a_row) * LDK + a_col;
            const float* qa = Qs + (16 * mi + a_row) * LDK + a_col;
            const float* kb = Ks + (8 * ni + (lane & 7)) * LDK + ((lane >> 3) & 1) * 4;
#pragma unroll 4
            for (int k0 = 0; k0 < DK; k0 += 8) {
                float fa[4], fq[4], fb[2];
                ldsm4(fa, ka + k0); ldsm4(fq, qa + k0); ldsm2(fb, kb + k0);
                mma_tf32(kk, fa[0], fa[1], fa[2], fa[3], fb[0], fb[1]);
                mma_tf32(qk, fq[0], fq[1], fq[2], fq[3], fb[0], fb[1]);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = 16 * mi + g + (e >> 1) * 8, jj = 8 * ni + 2 * t + (e & 1);
                const float dec = (jj <= i) ? __expf(Gs[i] - Gs[jj]) : 0.f;
                As[i * DC_LDA + jj] = (jj < i) ? bs[i] * dec * kk[e] : 0.f;
                Ws[i * DC_LDA + jj] = tf32r(dec * qk[e]);
            }
        }
        // tiles above the diagonal were not visited: they are zero
        for (int idx = tid; idx < DC_C * DC_C; idx += DN_THREADS) {
            const int i = idx / DC_C, jj = idx % DC_C;
            if ((jj >> 3) > ((i >> 4) * 2 + 1)) { As[i * DC_LDA + jj] = 0.f; Ws[i * DC_LDA + jj] = 0.f; }
        }
    }
    __syncthreads();
    if (kr == 0) {
        // column `lane` of T: t_i = [i == lane] - sum_{j < i} A_ij t_j
        float tc[DC_C];
#pragma unroll
        for (int i = 0; i < DC_C; ++i) {
            float v = (i == lane) ? 1.f : 0.f;
#pragma unroll
            for (int jj = 0; jj < DC_C; ++jj)
                if (jj < i) v = fmaf(-As[i * DC_LDA + jj], tc[jj], v);
            tc[i] = v;
            Ts[i * DC_LDA + lane] = v;
        }
    }
    __syncthreads();
    float* dst = tw + ((size_t)j * n_chunks + ci) * 2 * DC_C * DC_C;
    for (int idx = tid; idx < 2 * DC_C * DC_C; idx += DN_THREADS) {
        const int mat = idx / (DC_C * DC_C), rem = idx % (DC_C * DC_C);
        dst[idx] = (mat ? Ws : Ts)[(rem / DC_C) * DC_LDA + rem % DC_C];
    }
}

template <int DK, int DV>
static int launch_delta_chunk(const DeltaParams* p, const void* ab, int ld_ab, __half* qk_pre, int ld_qk, int n_rows,
                              float* tw, cudaStream_t s) {
    if (qk_pre) {
        dim3 grid((n_rows + QP_ROWS - 1) / QP_ROWS, p->nk);
        deltanet_qk_prep_kernel<DK><<<grid, 2 * DK, 0, s>>>(*p, qk_pre, ld_qk, DV / DN_COLS, 2 * DK + DN_COLS);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    const int n_chunks = (n_rows + DC_C - 1) / DC_C;
    if (qk_pre && tw) {
        const size_t psm = (size_t)(2 * DC_C * DC_LDK(DK) + 3 * DC_C * DC_LDA + 3 * DC_C) * sizeof(float);
        static SmemOptIn opt_tw;
        if (int e = opt_tw.ensure(deltanet_tw_prep_kernel<DK>, psm)) return e;
        deltanet_tw_prep_kernel<DK><<<dim3(n_chunks, p->nv), DN_THREADS, psm, s>>>(*p, (const __half*)ab, ld_ab, qk_pre, ld_qk, tw, n_chunks);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    } else {
        tw = nullptr;
    }
    constexpr int CB = DV / DN_COLS;
    constexpr int NCH = 2 * DK + DN_COLS;
    size_t smem = (size_t)(2 * DC_C * DC_LDK(DK) + DC_C * DC_LDU + 2 * DC_C * DN_COLS + 4 * DC_C * DC_LDA + DN_COLS * DC_LDK(DK) + NCH * 7 +
                           3 * DC_C + 2 * DC_C) * sizeof(float) + (size_t)(DC_C + 3) * NCH * sizeof(__half);
    static SmemOptIn optin;
    {
        cudaError_t e = optin.ensure(deltanet_chunk_kernel<DK, DV>, smem);
        if (e != cudaSuccess) return e;
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
    return cudaLaunchKernelEx(&cfg, deltanet_chunk_kernel<DK, DV>, *p, (const __half*)ab, ld_ab, (const __half*)qk_pre, ld_qk,
                              (const float*)tw, n_chunks);
}

// ab: [rows][ld_ab] fp16 with a at column head and b at column nv + head.
// qk_scratch (optional): fp16 [n_rows][ld_qk >= 2 * nk * dk] work buffer; with it, and ONE launched sequence of
// n_rows rows, the q / k convolution and norms run once in a parallel pre-pass instead of inside the scan.
// tw_scratch (optional, needs qk_scratch): fp32 [nv][ceil(n_rows / 32)][2][32][32]; with it the state-independent
// products of every chunk and the inverse of its triangle are computed in a second parallel pre-pass.
B2_API int b2_deltanet_chunk(const DeltaParams* p, const void* ab, int ld_ab, void* qk_scratch, int ld_qk, int n_rows,
                             void* tw_scratch, int dk, int dv, cudaStream_t s) {
    if (p->nv % p->nk || !ab) return cudaErrorInvalidValue;
    __half* qk = (__half*)qk_scratch;
    if (qk && (p->n_seqs != 1 || n_rows < 1 || ld_qk < 2 * p->nk * dk || (ld_qk & 7) || ((uintptr_t)qk & 15))) qk = nullptr;
    float* tw = (float*)tw_scratch;
    if (tw && (!qk || ((uintptr_t)tw & 15))) tw = nullptr;
    if (dk == 128 && dv == 128) return launch_delta_chunk<128, 128>(p, ab, ld_ab, qk, ld_qk, n_rows, tw, s);
    if (dk == 64 && dv == 64) return launch_delta_chunk<64, 64>(p, ab, ld_ab, qk, ld_qk, n_rows, tw, s);
    return cudaErrorInvalidValue;
}
B2_API long long b2_deltanet_tw_floats(int nv, int n_rows) { return (long long)nv * ((n_rows + DC_C - 1) / DC_C) * 2 * DC_C * DC_C; }

// a/b projections for many rows: ab[r][o] = x[r] . w[o], o < 2 nv (tiny dense weights).  A CTA stages
// AB_ROWS activation rows in shared memory and computes 8 outputs (one per warp) for all of them:
// grid = (row groups, output groups).
#define AB_ROWS 8
__global__ void __launch_bounds__(256) ab_proj_kernel(const __half* __restrict__ x, int ldx, const __half* __restrict__ wa,
                                                      const __half* __restrict__ wb, int nv, int H,
                                                      __half* __restrict__ ab, int ld_ab, int rows) {
    extern __shared__ __align__(16) __half xs[];           // [AB_ROWS][H]
    pdl_launch_dependents();
    const int r0 = blockIdx.x * AB_ROWS, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nr = min(AB_ROWS, rows - r0);
    for (int i = tid * 8; i < AB_ROWS * H; i += 256 * 8) {
        const int r = i / H, c = i - r * H;
        *(uint4*)(xs + i) = r < nr ? *(const uint4*)(x + (size_t)(r0 + r) * ldx + c) : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    for (int o = blockIdx.y * 8 + warp; o < min(2 * nv, (int)blockIdx.y * 8 + 8); o += 8) {
        const __half* w = (o < nv) ? wa + (size_t)o * H : wb + (size_t)(o - nv) * H;
        float acc[AB_ROWS];
#pragma unroll
        for (int r = 0; r < AB_ROWS; ++r) acc[r] = 0.f;
        for (int i = lane * 8; i < H; i += 256) {
            const uint4 wv = *(const uint4*)(w + i);
            const __half2* w2 = (const __half2*)&wv;
            float2 wf[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) wf[q] = __half22float2(w2[q]);
#pragma unroll
            for (int r = 0; r < AB_ROWS; ++r) {
                const uint4 xv = *(const uint4*)(xs + r * H + i);
                const __half2* x2 = (const __half2*)&xv;
#pragma unroll
                for (int q = 0; q < 4; ++q) { const float2 b = __half22float2(x2[q]); acc[r] += wf[q].x * b.x + wf[q].y * b.y; }
            }
        }
#pragma unroll
        for (int r = 0; r < AB_ROWS; ++r) {
            const float v = warp_sum(acc[r]);
            if (lane == 0 && r < nr) ab[(size_t)(r0 + r) * ld_ab + o] = __float2half(v);
        }
    }
}
B2_API int b2_ab_proj(const void* x, int ldx, const void* wa, const void* wb, int nv, int H, void* ab, int ld_ab,
                      int rows, cudaStream_t s) {
    if (H % 8 || (ldx % 8)) return cudaErrorInvalidValue;
    const size_t smem = (size_t)AB_ROWS * H * 2;
    static SmemOptIn optin;
    {
        cudaError_t e = optin.ensure(ab_proj_kernel, smem);
        if (e != cudaSuccess) return e;
    }
    ab_proj_kernel<<<dim3((rows + AB_ROWS - 1) / AB_ROWS, (2 * nv + 7) / 8), 256, smem, s>>>((const __half*)x, ldx, (const __half*)wa,
                                                                     (const __half*)wb, nv, H, (__half*)ab, ld_ab, rows);
    return cudaGetLastError();
}
