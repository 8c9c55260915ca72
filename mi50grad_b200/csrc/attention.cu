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
// head (GQA), so K/V are read once per group.  Each warp takes batches of cache
// slots whose rows are all requested before any is used, lanes split the head
// dimension (HD/32 elements each), scores are reduced with shuffles, and
// (max, sum, acc) are merged across warps in shared memory and across splits
// through a scratch buffer by the last CTA to arrive.
#include "kernels.cuh"

#define ATT_WARPS 8
#define ATT_THREADS (ATT_WARPS * 32)
#define ATT_MAX_G 8
#define ATT_BATCH 8              // cache slots a warp has in flight
#define ATT_GROUP 4              // slots per soft-max update
#define ATT_MIN_SPLIT_LEN (ATT_WARPS * ATT_BATCH)      // one pass of one CTA

// HD / 32 fp16 values of one cache row held by one lane
template <int EPL>
struct KVecT {
    uint32_t w[EPL / 2];
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < EPL / 2; ++i) w[i] = 0u;
    }
    __device__ __forceinline__ void load(const __half* p) {
        if constexpr (EPL == 8) { uint4 v = *(const uint4*)p; w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
        else if constexpr (EPL == 4) { uint2 v = *(const uint2*)p; w[0] = v.x; w[1] = v.y; }
        else { w[0] = *(const uint32_t*)p; }
    }
    __device__ __forceinline__ float get(int e) const {
        const __half2 h = *(const __half2*)&w[e >> 1];
        return (e & 1) ? __high2float(h) : __low2float(h);
    }
};


// GT: compile-time bound of the query heads per KV head (registers are sized by it).
template <int HD, int GT>
__global__ void __launch_bounds__(ATT_THREADS) decode_attn_kernel(const AttnParams p) {
    constexpr int EPL = HD / 32;                 // elements per lane
    using KVec = KVecT<EPL>;
    constexpr int LB = EPL * 2;                  // bytes of a cache row held by one lane
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
    // dynamic shared memory: during the walk over the cache a ring of K/V rows per warp
    // [2 stages][ATT_WARPS][ATT_BATCH][K | V][32 lanes][LB bytes]; afterwards the merge buffer [ATT_WARPS][G][HD]
    extern __shared__ __align__(16) unsigned char att_smem[];
    float* sm_acc = (float*)att_smem;
    unsigned char* ring = att_smem + ((size_t)warp * ATT_BATCH * 2 * 32 + lane) * LB;     // this lane's first entry
    constexpr size_t STAGE_B = (size_t)ATT_WARPS * ATT_BATCH * 2 * 32 * LB;
    __shared__ int s_last;
    __shared__ float sm_f[32][ATT_MAX_G], sm_ls[32][ATT_MAX_G], sm_linv[ATT_MAX_G];

    float q[GT][EPL], acc[GT][EPL], m[GT], l[GT];
#pragma unroll
    for (int h = 0; h < GT; ++h) {
        m[h] = -INFINITY; l[h] = 0.f;
        KVec qv;
        qv.zero();
        if (h < G) qv.load(p.q + (size_t)r * p.ldq + (kvh * G + h) * HD + lane * EPL);
#pragma unroll
        for (int e = 0; e < EPL; ++e) { acc[h][e] = 0.f; q[h][e] = qv.get(e) * p.scale; }
    }
    const size_t base = ((size_t)rm.seq * p.max_seq) * p.nkv * HD + (size_t)kvh * HD + lane * EPL;
    const size_t stride = (size_t)p.nkv * HD;
    // A warp takes ATT_BATCH cache slots at a time (slot = sb + i * ATT_WARPS + warp).  Their K and V rows
    // travel by cp.async into the warp's ring (each lane copies, and later reads back, only its own bytes, so
    // no barrier is involved), and the rows of the next batch are already on their way while this one is
    // processed: a pass costs no exposed trip to memory.  The scores of ATT_GROUP slots go through the
    // soft-max update together.
    auto issue = [&](int sb, int stage) {
#pragma unroll
        for (int i = 0; i < ATT_BATCH; ++i) {
            const int s = sb + i * ATT_WARPS + warp;
            if (s < s1) {
                unsigned char* dst = ring + stage * STAGE_B + (size_t)i * 2 * 32 * LB;
                const __half* kp = p.kcache + base + (size_t)s * stride;
                const __half* vp = p.vcache + base + (size_t)s * stride;
                if constexpr (LB == 16) { cp_async16(dst, kp); cp_async16(dst + 32 * LB, vp); }
                else if constexpr (LB == 8) { cp_async8(dst, kp); cp_async8(dst + 32 * LB, vp); }
                else { cp_async4(dst, kp); cp_async4(dst + 32 * LB, vp); }
            }
        }
        cp_async_commit();
    };
    constexpr int PASS = ATT_WARPS * ATT_BATCH;
    if (s0 < s1) issue(s0, 0);
    int stage = 0;
    for (int sb = s0; sb < s1; sb += PASS, stage ^= 1) {
        if (sb + PASS < s1) { issue(sb + PASS, stage ^ 1); cp_async_wait<1>(); }
        else cp_async_wait<0>();
#pragma unroll 1
        for (int g0 = 0; g0 < ATT_BATCH; g0 += ATT_GROUP) {
            if (sb + g0 * ATT_WARPS + warp >= s1) break;       // uniform per warp: slots grow with i
            const unsigned char* src = ring + stage * STAGE_B + (size_t)g0 * 2 * 32 * LB;
            float d[ATT_GROUP][GT];
            bool vis[ATT_GROUP];
#pragma unroll
            for (int i = 0; i < ATT_GROUP; ++i) {
                const int s = sb + (g0 + i) * ATT_WARPS + warp;
                vis[i] = s < s1 && (s < rm.ctx || ((rm.mask >> (s - rm.ctx)) & 1ull));
                KVec kk;
                kk.zero();
                if (s < s1) kk.load((const __half*)(src + (size_t)i * 2 * 32 * LB));
                float kf[EPL];
#pragma unroll
                for (int e = 0; e < EPL; ++e) kf[e] = kk.get(e);
#pragma unroll
                for (int h = 0; h < GT; ++h) {
                    float x = 0.f;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) x = fmaf(q[h][e], kf[e], x);
                    d[i][h] = x;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int i = 0; i < ATT_GROUP; ++i)
#pragma unroll
                    for (int h = 0; h < GT; ++h) d[i][h] += __shfl_xor_sync(0xffffffffu, d[i][h], o);
            float vf[ATT_GROUP][EPL];
#pragma unroll
            for (int i = 0; i < ATT_GROUP; ++i) {
                KVec vv;
                vv.zero();
                if (sb + (g0 + i) * ATT_WARPS + warp < s1) vv.load((const __half*)(src + ((size_t)i * 2 + 1) * 32 * LB));
#pragma unroll
                for (int e = 0; e < EPL; ++e) vf[i][e] = vv.get(e);
            }
#pragma unroll
            for (int h = 0; h < GT; ++h) {
                float mn = m[h];
#pragma unroll
                for (int i = 0; i < ATT_GROUP; ++i) if (vis[i]) mn = fmaxf(mn, d[i][h]);
                if (mn == -INFINITY) continue;                 // nothing visible so far
                const float corr = __expf(m[h] - mn);          // exp(-inf) = 0 on the first visible slot
                float pw[ATT_GROUP], ps = 0.f;
#pragma unroll
                for (int i = 0; i < ATT_GROUP; ++i) { pw[i] = vis[i] ? __expf(d[i][h] - mn) : 0.f; ps += pw[i]; }
                l[h] = l[h] * corr + ps;
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    float a = acc[h][e] * corr;
#pragma unroll
                    for (int i = 0; i < ATT_GROUP; ++i) a = fmaf(pw[i], vf[i][e], a);
                    acc[h][e] = a;
                }
                m[h] = mn;
            }
        }
    }
    __syncthreads();                             // every warp is done with its ring: the merge buffer reuses it
    // ---- merge the warps of this CTA
#pragma unroll
    for (int h = 0; h < GT; ++h) {
        if (h < G) {
            if (lane == 0) { sm_m[warp][h] = m[h]; sm_l[warp][h] = l[h]; }
#pragma unroll
            for (int e = 0; e < EPL; ++e) sm_acc[((size_t)warp * G + h) * HD + lane * EPL + e] = acc[h][e];
        }
    }
    __syncthreads();
    // thread tid handles (h, d) pairs
    float* my = p.scratch + (((size_t)r * p.nkv + kvh) * p.splits + sp) * G * (HD + 4);
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
            a += sm_acc[((size_t)w * G + h) * HD + d] * f;
        }
        if (nsplit == 1) {
            float o = ll > 0.f ? a / ll : 0.f;
            size_t col = (size_t)(kvh * G + h) * HD + d;
            if (p.gate_off >= 0) o *= sigmoid_f(__half2float(p.q[(size_t)r * p.ldq + p.gate_off + col]));
            p.out[(size_t)r * p.ldo + col] = __float2half(o);
        } else {
            my[h * (HD + 4) + d] = a;
            if (d == 0) { my[h * (HD + 4) + HD] = mm; my[h * (HD + 4) + HD + 1] = ll; }
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
    const float* all = p.scratch + (((size_t)r * p.nkv + kvh) * splits_orig) * G * (HD + 4);
    // phase 1: per (split, head) rescale factors, one round trip
    for (int idx = tid; idx < nsplit * G; idx += ATT_THREADS) {
        int s = idx / G, h = idx % G;
        const float* e = &all[(size_t)(s * G + h) * (HD + 4)];
        sm_f[s][h] = ld_cg_f32(e + HD);                 // max of split s
        sm_ls[s][h] = ld_cg_f32(e + HD + 1);            // its sum
    }
    __syncthreads();
    if (tid < G) {
        float mm = -INFINITY;
        for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, sm_f[s][tid]);
        float ll = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            float f = (sm_f[s][tid] == -INFINITY) ? 0.f : __expf(sm_f[s][tid] - mm);
            ll += sm_ls[s][tid] * f;
            sm_f[s][tid] = f;
        }
        sm_linv[tid] = ll > 0.f ? 1.f / ll : 0.f;
    }
    __syncthreads();
    // phase 2: weighted sum of the partial outputs, four columns per thread; the loads of up to eight splits
    // are issued together (a loop of load-then-accumulate would wait for every load in turn)
    for (int i = tid; i < G * (HD / 4); i += ATT_THREADS) {
        const int h = i / (HD / 4), d = (i % (HD / 4)) * 4;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sb = 0; sb < nsplit; sb += 8) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                v[u] = (sb + u < nsplit) ? ld_cg_v4(&all[(size_t)((sb + u) * G + h) * (HD + 4) + d]) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float f = (sb + u < nsplit) ? sm_f[sb + u][h] : 0.f;
                a.x += v[u].x * f; a.y += v[u].y * f; a.z += v[u].z * f; a.w += v[u].w * f;
            }
        }
        const float li = sm_linv[h];
        const size_t col = (size_t)(kvh * G + h) * HD + d;
        float o[4] = {a.x * li, a.y * li, a.z * li, a.w * li};
        if (p.gate_off >= 0) {
            const uint2 gq = *(const uint2*)(p.q + (size_t)r * p.ldq + p.gate_off + col);
            const float2 g0 = __half22float2(*(const __half2*)&gq.x), g1 = __half22float2(*(const __half2*)&gq.y);
            o[0] *= sigmoid_f(g0.x); o[1] *= sigmoid_f(g0.y); o[2] *= sigmoid_f(g1.x); o[3] *= sigmoid_f(g1.y);
        }
        __half2 o01 = __floats2half2_rn(o[0], o[1]), o23 = __floats2half2_rn(o[2], o[3]);
        uint2 st;
        st.x = *(uint32_t*)&o01; st.y = *(uint32_t*)&o23;
        *(uint2*)(p.out + (size_t)r * p.ldo + col) = st;
    }
}

template <int HD, int GT>
static int launch_decode_attn(const AttnParams* p, cudaStream_t s) {
    dim3 grid(p->nkv, p->n_rows, p->splits);
    const size_t ring = (size_t)2 * ATT_WARPS * ATT_BATCH * 2 * HD * sizeof(__half);
    const size_t merge = (size_t)ATT_WARPS * (p->nq / p->nkv) * HD * sizeof(float);
    const size_t smem = ring > merge ? ring : merge;
    static SmemOptIn opt;
    if (int e = opt.ensure((const void*)decode_attn_kernel<HD, GT>, smem)) return e;
    return launch_pdl(decode_attn_kernel<HD, GT>, grid, dim3(ATT_THREADS), smem, s, *p);
}
template <int HD>
static int launch_decode_attn_g(const AttnParams* p, int G, cudaStream_t s) {
    if (G <= 1) return launch_decode_attn<HD, 1>(p, s);
    if (G <= 2) return launch_decode_attn<HD, 2>(p, s);
    if (G <= 3) return launch_decode_attn<HD, 3>(p, s);
    if (G <= 4) return launch_decode_attn<HD, 4>(p, s);
    if (G <= 6) return launch_decode_attn<HD, 6>(p, s);
    return launch_decode_attn<HD, 8>(p, s);
}

B2_API int b2_decode_attn(const AttnParams* p, int hd, cudaStream_t s) {
    if (p->nq % p->nkv || p->nq / p->nkv > ATT_MAX_G || p->splits < 1 || p->splits > 32) return cudaErrorInvalidValue;
    const int G = p->nq / p->nkv;
    if (hd == 256) return launch_decode_attn_g<256>(p, G, s);
    if (hd == 128) return launch_decode_attn_g<128>(p, G, s);
    if (hd == 64) return launch_decode_attn_g<64>(p, G, s);
    return cudaErrorInvalidValue;
}
B2_API int b2_sizeof_attn_params() { return (int)sizeof(AttnParams); }
