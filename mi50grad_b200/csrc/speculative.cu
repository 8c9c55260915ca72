// Speculative verification on the device: draft chains or trees are checked in ONE
// forward pass and the sequence state afterwards is exactly what feeding only the
// accepted tokens would have produced.
//
// The reference accepts drafts on the host, token by token, and its rollback only
// rewinds a length counter, so rejected drafts stay in the DeltaNet state; its tree
// pass gives every node RoPE position 0 and lets the DeltaNet layers ignore the tree
// (reference: src/inference/speculative.py:231-417, src/inference/tree_speculative.py:296-383,
// src/inference/tp_engine.py:1673-1687,3170-3236).
//
// Four kernels:
//  * deltanet_verify: Gated DeltaNet over a draft tree WITHOUT touching the state.  With S0
//    the committed state, G_t the summed log-decay along node t's path and u_t its rank-1
//    update vector, the state after any path is
//        S_path = exp(G_last) S0 + sum_{a in path} exp(G_last - G_a) k_a u_a^T,
//    so every node needs S0 only through S0^T k_t and S0^T q_t (one pass over the state in
//    registers) plus dot products with its ancestors' keys.  The kernel stages k, u, G and
//    the raw conv inputs of every node for the commit.
//  * spec_accept: greedy acceptance.  Walks the tree from the pending token, following the
//    child whose token equals the model's prediction, advances the sequence length and
//    stores the next pending token.
//  * deltanet_commit: applies the accepted path's rank-1 updates and conv inputs to the
//    state of every linear-attention layer in one launch.
//  * kv_compact: moves the accepted nodes' K/V from slot len+node to slot len+depth in every
//    full-attention layer (a no-op for chains).
#include <cooperative_groups.h>
#include "kernels.cuh"
namespace cg = cooperative_groups;

#define DN_THREADS 256
#define DN_COLS 32
#define NM SPEC_MAX_NODES

__device__ __forceinline__ int top_bit(unsigned m) { return m ? 31 - __clz(m) : -1; }

template <int DK, int DV>
__global__ void __launch_bounds__(DN_THREADS) deltanet_verify_kernel(const DeltaParams p, const SpecStage st,
                                                                      int layer) {
    constexpr int CB = DV / DN_COLS;
    constexpr int RPT = DK / 8;
    constexpr int NCH = 2 * DK + DN_COLS;
    cg::cluster_group cluster = cg::this_cluster();
    pdl_launch_dependents();
    const int cb = blockIdx.x, j = blockIdx.y, si = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, kr = tid >> 5, vcol = lane;
    const int rep = p.nv / p.nk, kh = j / rep;
    const int r0 = p.seq_rows[si], r1 = p.seq_rows[si + 1];
    if (r0 >= r1) return;                        // uniform over the whole cluster
    const int N = min(r1 - r0, NM);
    const int seq = p.rows[r0].seq;

    __shared__ float hist[NCH][3];
    __shared__ float cw[NCH][4];
    __shared__ __half xraw[NM][NCH];
    __shared__ float khat[NM][DK];
    __shared__ float uu[NM][DN_COLS], yy[NM][DN_COLS];
    __shared__ float Gs[NM], dkk[NM], dkq[NM];
    __shared__ float cq[DK], ck[DK], cv[DN_COLS];
    __shared__ float red_m[8][DN_COLS], red_q[8][DN_COLS];
    __shared__ float red32[8];
    __shared__ float cl_ss[NM];

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
    const __half* my_hist = p.conv_state + ((((size_t)seq * p.nv + j) * CB + cb) * NCH) * 3;
    for (int c = tid; c < NCH; c += DN_THREADS) {
#pragma unroll
        for (int t = 0; t < 3; ++t) hist[c][t] = __half2float(my_hist[c * 3 + t]);
        const __half* w = p.conv_w + (size_t)chan(c) * 4;
#pragma unroll
        for (int t = 0; t < 4; ++t) cw[c][t] = __half2float(w[t]);
    }
    float S[RPT];
    const float* sp = p.state + (((size_t)seq * p.nv + j) * DK) * DV + cb * DN_COLS + vcol;
#pragma unroll
    for (int i = 0; i < RPT; ++i) S[i] = sp[(size_t)(kr + 8 * i) * DV];
    const float neg_expA = -__expf(p.A_log[j]);
    const float dtb = __half2float(p.dt_bias[j]);
    const float nw = __half2float(p.norm_w[cb * DN_COLS + vcol]);
    const bool inkernel_ab = p.off_a < 0;
    __syncthreads();

    for (int t = 0; t < N; ++t) {
        const int r = r0 + t;
        const __half* pr = p.proj + (size_t)r * p.ld;
        // ancestors of node t inside this sequence's block (bit a <-> node a), nearest first
        const unsigned anc = (unsigned)(p.rows[r].mask & 0xFFFFull) & ((1u << t) - 1u);
        const int d = __popc(anc);
        const int p1 = top_bit(anc);
        const unsigned a2 = p1 >= 0 ? anc & ~(1u << p1) : 0u;
        const int p2 = top_bit(a2);
        const int p3 = top_bit(p2 >= 0 ? a2 & ~(1u << p2) : 0u);
        // ---- phase A: a/b partial sums, conv + SiLU along the node's path
        float sa = 0.f, sb = 0.f;
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
            const __half xh = pr[proj_col(c)];
            xraw[t][c] = xh;
            const float x = __half2float(xh);
            // taps at distance 1..3 along the path; beyond the root they come from the history
            const float x1 = d >= 1 ? __half2float(xraw[p1][c]) : hist[c][2];
            const float x2 = d >= 2 ? __half2float(xraw[p2][c]) : hist[c][1 + d];
            const float x3 = d >= 3 ? __half2float(xraw[p3][c]) : hist[c][d];
            float o = x3 * cw[c][0] + x2 * cw[c][1] + x1 * cw[c][2] + x * cw[c][3];
            o = silu_f(o);
            if (c < DK) cq[c] = o; else if (c < 2 * DK) ck[c - DK] = o; else cv[c - 2 * DK] = o;
        }
        __syncthreads();
        // ---- phase B: norms, q.k, and the dot products with every ancestor's key
        for (int idx = kr; idx < 3 + 2 * d; idx += 8) {
            float s = 0.f;
            if (idx < 3) {
                for (int i = lane; i < DK; i += 32) {
                    float a = (idx == 1) ? ck[i] : cq[i], b = (idx == 0) ? cq[i] : ck[i];
                    s += a * b;                  // 0: q.q  1: k.k  2: q.k
                }
                s = warp_sum(s);
                if (lane == 0) red32[idx] = s;
            } else {
                int ord = (idx - 3) >> 1;
                unsigned m = anc;
                for (int q = 0; q < ord; ++q) m &= m - 1;          // drop the `ord` lowest ancestors
                const int a = __ffs(m) - 1;
                const float* other = ((idx - 3) & 1) ? cq : ck;
                for (int i = lane; i < DK; i += 32) s += khat[a][i] * other[i];
                s = warp_sum(s);
                if (lane == 0) { if ((idx - 3) & 1) dkq[a] = s; else dkk[a] = s; }
            }
        }
        if (kr == 7) {
            float a_in, b_in;
            if (inkernel_ab) {
                float inv = p.ln.h ? lazy_inv_rms(p.ln, r, lane) : 1.f;
                float ta = 0.f, tb = 0.f;
#pragma unroll
                for (int w = 0; w < 8; ++w) { ta += red_m[w][0]; tb += red_m[w][1]; }
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
        const float Gp = p1 >= 0 ? Gs[p1] : 0.f;
        const float Gt = Gp + gl;
        // ---- phase C: S0^T k and S0^T q for this CTA's columns
        float mp = 0.f, qp = 0.f;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            mp = fmaf(S[i], ck[kr + 8 * i], mp);
            qp = fmaf(S[i], cq[kr + 8 * i], qp);
        }
        red_m[kr][vcol] = mp * invk;
        red_q[kr][vcol] = qp * invq;
        for (int i = tid; i < DK; i += DN_THREADS) khat[t][i] = ck[i] * invk;
        __syncthreads();
        float mm = 0.f, sq = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) { mm += red_m[w][vcol]; sq += red_q[w][vcol]; }
        float Sk = __expf(Gp) * mm;              // S_parent^T k_t
        float ys = __expf(Gt) * sq;              // decayed S0 part of S_t^T q_t
        for (unsigned m = anc; m; m &= m - 1) {
            const int a = __ffs(m) - 1;
            const float ua = uu[a][vcol], Ga = Gs[a];
            Sk = fmaf(__expf(Gp - Ga) * ua, dkk[a] * invk, Sk);
            ys = fmaf(__expf(Gt - Ga) * ua, dkq[a] * invq, ys);
        }
        const float delta = (cv[vcol] - decay * Sk) * beta;
        const float y = ys + delta * kq;
        const float ss = warp_sum(y * y);
        __syncthreads();                          // all reads of Gs/uu/red_* of this node are done
        if (kr == 0) { uu[t][vcol] = delta; yy[t][vcol] = y; }
        if (tid == 0) { cl_ss[t] = ss; Gs[t] = Gt; }
        __syncthreads();
    }
    cluster.sync();
    // ---- gated RMSNorm over the head's dv outputs, one warp per node
    for (int t = kr; t < N; t += 8) {
        float tot = 0.f;
#pragma unroll
        for (int c = 0; c < CB; ++c) tot += *cluster.map_shared_rank(&cl_ss[t], c);
        const __half* pr = p.proj + (size_t)(r0 + t) * p.ld;
        const float z = __half2float(pr[p.off_z + j * DV + cb * DN_COLS + vcol]);
        const float o = yy[t][vcol] * rsqrtf(tot / (float)DV + p.eps) * nw * silu_f(z);
        p.out[(size_t)(r0 + t) * p.ldo + j * DV + cb * DN_COLS + vcol] = __float2half(o);
    }
    // ---- staging for the commit
    unsigned char* blk = st.base + (size_t)layer * st.layer_stride + (size_t)si * st.seq_stride;
    float* su = (float*)(blk + st.off_u);
    for (int t = kr; t < N; t += 8) su[((size_t)t * p.nv + j) * DV + cb * DN_COLS + vcol] = uu[t][vcol];
    const int conv_dim = 2 * p.nk * DK + p.nv * DV;
    __half* sx = (__half*)(blk + st.off_x);
    const bool key_owner = (cb == 0) && (j % rep == 0);
    for (int i = tid; i < N * NCH; i += DN_THREADS) {
        const int t = i / NCH, c = i - t * NCH;
        if (c >= 2 * DK || key_owner) sx[(size_t)t * conv_dim + chan(c)] = xraw[t][c];
    }
    if (cb == 0 && tid < N) ((float*)(blk + st.off_g))[tid * p.nv + j] = Gs[tid];
    if (key_owner) {
        float* sk = (float*)(blk + st.off_k);
        for (int i = tid; i < N * DK; i += DN_THREADS) {
            const int t = i / DK, e = i - t * DK;
            sk[((size_t)t * p.nk + kh) * DK + e] = khat[t][e];
        }
    }
    cluster.sync();                              // no CTA leaves while a peer may still read its shared memory
}

template <int DK, int DV>
static int launch_verify(const DeltaParams* p, const SpecStage* st, int layer, cudaStream_t s) {
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
    return cudaLaunchKernelEx(&cfg, deltanet_verify_kernel<DK, DV>, *p, *st, layer);
}

B2_API int b2_deltanet_verify(const DeltaParams* p, const SpecStage* st, int layer, int dk, int dv, cudaStream_t s) {
    if (p->nv % p->nk || !st->base) return cudaErrorInvalidValue;
    if (dk == 128 && dv == 128) return launch_verify<128, 128>(p, st, layer, s);
    if (dk == 64 && dv == 64) return launch_verify<64, 64>(p, st, layer, s);
    return cudaErrorInvalidValue;
}

// Bytes of one staging block and its section offsets.
B2_API long long b2_spec_stage_layout(int nk, int nv, int dk, int dv, int* off_k, int* off_u, int* off_g, int* off_x) {
    auto al = [](long long x) { return (x + 255) & ~255LL; };
    long long o = 0;
    *off_k = (int)o; o = al(o + (long long)NM * nk * dk * 4);
    *off_u = (int)o; o = al(o + (long long)NM * nv * dv * 4);
    *off_g = (int)o; o = al(o + (long long)NM * nv * 4);
    *off_x = (int)o; o = al(o + (long long)NM * (2LL * nk * dk + (long long)nv * dv) * 2);
    return o;
}

// ---------------------------------------------------------------------------
// spec_accept: one thread per sequence (a tree has at most 16 nodes).
// ---------------------------------------------------------------------------
__global__ void spec_accept_kernel(const SpecAcceptParams p) {
    pdl_launch_dependents();
    const int si = blockIdx.x * blockDim.x + threadIdx.x;
    if (si >= p.n_seqs) return;
    int* acc = p.acc + (size_t)si * (NM + 2);
    int* res = p.result + (size_t)si * (NM + 2);
    const int r0 = p.seq_rows[si], r1 = p.seq_rows[si + 1];
    const int N = min(r1 - r0, NM);
    if (N <= 0) { acc[0] = 0; res[0] = -1; return; }
    int parent[NM];
    for (int t = 0; t < N; ++t)
        parent[t] = top_bit((unsigned)(p.rows[r0 + t].mask & 0xFFFFull) & ((1u << t) - 1u));
    int cur = 0, n = 1;
    acc[1] = p.rows[r0].slot;                    // cache slot of the root = length before this step
    acc[2] = 0;
    for (;;) {
        const int pred = p.out_tokens[r0 + cur];
        int nxt = -1;
        for (int t = cur + 1; t < N; ++t)
            if (parent[t] == cur && p.row_tokens[r0 + t] == pred) { nxt = t; break; }
        if (nxt < 0) break;
        res[2 + n - 1] = pred;
        acc[2 + n] = nxt;
        ++n;
        cur = nxt;
    }
    const int next_tok = p.out_tokens[r0 + cur];
    acc[0] = n;
    res[0] = n - 1;
    res[1] = next_tok;
    SeqState* s = p.seqs + p.rows[r0].seq;
    s->len += n;
    s->token = next_tok;
}

B2_API int b2_spec_accept(const SpecAcceptParams* p, cudaStream_t s) {
    if (p->n_seqs < 1) return cudaErrorInvalidValue;
    spec_accept_kernel<<<(p->n_seqs + 31) / 32, 32, 0, s>>>(*p);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// deltanet_commit: grid (dv/32, v heads, layers * sequences)
// ---------------------------------------------------------------------------
template <int DK, int DV>
__global__ void __launch_bounds__(DN_THREADS) deltanet_commit_kernel(const DeltaCommitParams p) {
    constexpr int CB = DV / DN_COLS;
    constexpr int RPT = DK / 8;
    constexpr int NCH = 2 * DK + DN_COLS;
    pdl_launch_dependents();
    const int cb = blockIdx.x, j = blockIdx.y;
    const int layer = blockIdx.z / p.n_seqs, si = blockIdx.z - layer * p.n_seqs;
    const int tid = threadIdx.x, lane = tid & 31, kr = tid >> 5, vcol = lane;
    const int rep = p.nv / p.nk, kh = j / rep;
    const int* acc = p.acc + (size_t)si * (NM + 2);
    const int n = acc[0];
    if (n <= 0) return;
    const int seq = p.rows[p.seq_rows[si]].seq;
    const unsigned char* blk = p.st.base + (size_t)layer * p.st.layer_stride + (size_t)si * p.st.seq_stride;
    const float* sk = (const float*)(blk + p.st.off_k);
    const float* su = (const float*)(blk + p.st.off_u);
    const float* sg = (const float*)(blk + p.st.off_g);
    const __half* sx = (const __half*)(blk + p.st.off_x);

    __shared__ float kp[NM][DK];
    __shared__ float up[NM][DN_COLS];
    __shared__ float coef[NM];
    __shared__ int path[NM];
    if (tid < n) path[tid] = acc[2 + tid];
    __syncthreads();
    const float Gl = sg[path[n - 1] * p.nv + j];
    if (tid < n) coef[tid] = __expf(Gl - sg[path[tid] * p.nv + j]);
    for (int i = tid; i < n * DK; i += DN_THREADS) {
        const int a = i / DK, e = i - a * DK;
        kp[a][e] = sk[((size_t)path[a] * p.nk + kh) * DK + e];
    }
    for (int i = tid; i < n * DN_COLS; i += DN_THREADS) {
        const int a = i / DN_COLS, e = i - a * DN_COLS;
        up[a][e] = su[((size_t)path[a] * p.nv + j) * DV + cb * DN_COLS + e];
    }
    __syncthreads();
    float* sp = p.state0 + (size_t)layer * p.state_layer_stride + (((size_t)seq * p.nv + j) * DK) * DV +
                cb * DN_COLS + vcol;
    float S[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) S[i] = sp[(size_t)(kr + 8 * i) * DV];
    const float g0 = __expf(Gl);
#pragma unroll
    for (int i = 0; i < RPT; ++i) S[i] *= g0;
    for (int a = 0; a < n; ++a) {
        const float cu = coef[a] * up[a][vcol];
#pragma unroll
        for (int i = 0; i < RPT; ++i) S[i] = fmaf(kp[a][kr + 8 * i], cu, S[i]);
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) sp[(size_t)(kr + 8 * i) * DV] = S[i];
    // conv history: the last three inputs of [history, path inputs]
    __half* my_hist = p.conv0 + (size_t)layer * p.conv_layer_stride + ((((size_t)seq * p.nv + j) * CB + cb) * NCH) * 3;
    const int conv_dim = 2 * p.nk * DK + p.nv * DV;
    for (int c = tid; c < NCH; c += DN_THREADS) {
        int ch;
        if (c < DK) ch = kh * DK + c;
        else if (c < 2 * DK) ch = p.nk * DK + kh * DK + (c - DK);
        else ch = 2 * p.nk * DK + j * DV + cb * DN_COLS + (c - 2 * DK);
        __half h[3];
#pragma unroll
        for (int t = 0; t < 3; ++t) {
            const int pos = n + t;               // index into [h0 h1 h2 x_0 .. x_{n-1}], last three
            h[t] = pos < 3 ? my_hist[c * 3 + pos] : sx[(size_t)path[pos - 3] * conv_dim + ch];
        }
#pragma unroll
        for (int t = 0; t < 3; ++t) my_hist[c * 3 + t] = h[t];
    }
}

B2_API int b2_deltanet_commit(const DeltaCommitParams* p, int dk, int dv, cudaStream_t s) {
    if (p->nv % p->nk || p->n_layers < 1 || p->n_seqs < 1) return cudaErrorInvalidValue;
    dim3 grid(dv / DN_COLS, p->nv, p->n_layers * p->n_seqs);
    if (dk == 128 && dv == 128) deltanet_commit_kernel<128, 128><<<grid, DN_THREADS, 0, s>>>(*p);
    else if (dk == 64 && dv == 64) deltanet_commit_kernel<64, 64><<<grid, DN_THREADS, 0, s>>>(*p);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// kv_compact: grid (layers * kv heads, sequences); moves go in increasing depth, each
// destination slot is at or before its source, so earlier moves never clobber later sources.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) kv_compact_kernel(const KvCompactParams p) {
    pdl_launch_dependents();
    const int layer = blockIdx.x / p.nkv, kvh = blockIdx.x - layer * p.nkv, si = blockIdx.y;
    const int* acc = p.acc + (size_t)si * (NM + 2);
    const int n = acc[0];
    if (n <= 1) return;
    const int len0 = acc[1];
    const int seq = p.rows[p.seq_rows[si]].seq;
    const size_t base = (size_t)layer * p.layer_stride + ((size_t)seq * p.max_seq) * p.nkv * p.hd + (size_t)kvh * p.hd;
    const size_t stride = (size_t)p.nkv * p.hd;
    for (int d = 1; d < n; ++d) {
        const int t = acc[2 + d];
        if (t == d) continue;                    // uniform over the CTA
        const size_t src = base + (size_t)(len0 + t) * stride, dst = base + (size_t)(len0 + d) * stride;
        for (int e = threadIdx.x * 2; e < p.hd; e += 256) {
            *(__half2*)(p.k0 + dst + e) = *(const __half2*)(p.k0 + src + e);
            *(__half2*)(p.v0 + dst + e) = *(const __half2*)(p.v0 + src + e);
        }
        __syncthreads();
    }
}

B2_API int b2_kv_compact(const KvCompactParams* p, cudaStream_t s) {
    if (p->n_layers < 1 || p->n_seqs < 1 || (p->hd & 1)) return cudaErrorInvalidValue;
    dim3 grid(p->n_layers * p->nkv, p->n_seqs);
    kv_compact_kernel<<<grid, 128, 0, s>>>(*p);
    return cudaGetLastError();
}
B2_API int b2_sizeof_spec_stage() { return (int)sizeof(SpecStage); }
B2_API int b2_sizeof_spec_accept_params() { return (int)sizeof(SpecAcceptParams); }
B2_API int b2_sizeof_delta_commit_params() { return (int)sizeof(DeltaCommitParams); }
B2_API int b2_sizeof_kv_compact_params() { return (int)sizeof(KvCompactParams); }
