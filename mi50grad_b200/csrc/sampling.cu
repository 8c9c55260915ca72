// Greedy token selection on the device: two-stage arg-max over this rank's
// vocabulary slice, then a cross-rank arg-max through symmetric memory, so that
// logits never leave the GPU during decode (the reference downloads 248320
// logits per token and samples in numpy: src/inference/generate.py:126-145,
// src/inference/sampler.py:24-80).  Ties go to the lowest token id, which is
// what numpy.argmax returns.
#include "kernels.cuh"

__device__ __forceinline__ void arg_better(float& v, int& i, float v2, int i2) {
    if (v2 > v || (v2 == v && i2 < i)) { v = v2; i = i2; }
}

__global__ void __launch_bounds__(256) argmax_kernel(const ArgmaxParams p) {
    const int r = blockIdx.y, b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ int s_last, s_fail;
    const float* row = p.logits + (size_t)r * p.ld;
    const int per = (p.vocab_local + p.blocks - 1) / p.blocks;
    const int i0 = b * per, i1 = min(p.vocab_local, i0 + per);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = i0 + tid; i < i1; i += 256) arg_better(best, bi, row[i], i);
    auto block_arg = [&]() {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float v2 = __shfl_xor_sync(0xffffffffu, best, o);
            int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
            arg_better(best, bi, v2, i2);
        }
        __syncthreads();
        if (lane == 0) { sv[warp] = best; si[warp] = bi; }
        __syncthreads();
        best = sv[0]; bi = si[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) arg_better(best, bi, sv[w], si[w]);
    };
    block_arg();
    if (p.blocks > 1) {
        if (tid == 0) {
            float* s = p.scratch + ((size_t)r * p.blocks + b) * 2;
            s[0] = best;
            s[1] = __int_as_float(bi);
            __threadfence();
            int old = atomicAdd(&p.counters[r], 1);
            s_last = (old == p.blocks - 1);
            if (s_last) p.counters[r] = 0;
            __threadfence();
        }
        __syncthreads();
        if (!s_last) return;
        best = -INFINITY; bi = 0x7fffffff;
        for (int i = tid; i < p.blocks; i += 256) {
            const float* s = p.scratch + ((size_t)r * p.blocks + i) * 2;
            arg_better(best, bi, ld_cg_f32(s), __float_as_int(ld_cg_f32(s + 1)));
        }
        block_arg();
    }
    int token = bi + p.vocab_offset;
    // ---- cross-rank: rows are finished by different CTAs, so each row uses its own
    // slot and the exchange is done by row 0's CTA after all rows have arrived.
    const CommCtx& c = p.comm;
    if (c.tp > 1) {
        const uint32_t epoch_next = *c.epoch + 1u;
        float* mine = c.part[c.rank] + (size_t)(epoch_next & 1) * c.part_stride;
        if (tid == 0) {
            mine[2 * r] = best;
            mine[2 * r + 1] = __int_as_float(token);
            __threadfence();
            int old = atomicAdd(&p.counters[p.n_rows], 1);
            s_last = (old == p.n_rows - 1);
            if (s_last) p.counters[p.n_rows] = 0;
            __threadfence();
            s_fail = 0;
        }
        __syncthreads();
        if (!s_last) return;
        if (tid == 0) *c.epoch = epoch_next;
        if (tid < c.tp && tid != c.rank) {
            st_release_sys_u32(c.sig[tid] + c.rank, epoch_next);
            if (!wait_reached(c.sig[c.rank] + tid, epoch_next, c.wait_ns)) {
                report_timeout(c, B2_KID_ARGMAX, tid, epoch_next);
                s_fail = 1;
            }
        }
        __syncthreads();
        for (int rr = tid; rr < p.n_rows; rr += 256) {
            float v = -INFINITY;
            int t = 0x7fffffff;
            for (int pr = 0; pr < c.tp; ++pr) {
                if (s_fail && pr != c.rank) continue;
                const float* src = c.part[pr] + (size_t)(epoch_next & 1) * c.part_stride + 2 * rr;
                float2 e;
                asm volatile("ld.relaxed.sys.global.v2.f32 {%0,%1}, [%2];" : "=f"(e.x), "=f"(e.y) : "l"(src) : "memory");
                arg_better(v, t, e.x, __float_as_int(e.y));
            }
            p.out_tokens[rr] = t;
            if (p.seqs) p.seqs[p.rows[rr].seq].token = t;
        }
        return;
    }
    if (tid == 0) {
        p.out_tokens[r] = token;
        if (p.seqs) p.seqs[p.rows[r].seq].token = token;
    }
}

B2_API int b2_argmax(const ArgmaxParams* p, cudaStream_t s) {
    if (p->blocks < 1 || p->blocks > 1024) return cudaErrorInvalidValue;
    dim3 grid(p->blocks, p->n_rows);
    argmax_kernel<<<grid, 256, 0, s>>>(*p);
    return cudaGetLastError();
}
B2_API int b2_sizeof_argmax_params() { return (int)sizeof(ArgmaxParams); }

// ---------------------------------------------------------------------------
// Temperature / top-k / top-p sampling on the device, one CTA per row (the reference samples in
// numpy on the host after downloading the logits: src/inference/sampler.py:24-80).  Same pipeline:
// repetition penalty -> temperature -> top-k -> softmax -> top-p -> multinomial.
//   1. penalty on the row's past tokens (values are read first, then written, so duplicates in the
//      list count once);
//   2. the top-k threshold by bisection over the order-preserving integer image of the logits
//      (32 counting passes over the row, which stays in L2);
//   3. candidates above the threshold are gathered into shared memory (at most SAMPLE_MAX_CAND; with
//      top_k = 0 the SAMPLE_MAX_CAND most likely tokens stand in for the whole vocabulary), sorted
//      by (value descending, id ascending) with a bitonic network;
//   4. softmax at the given temperature, inclusive scan, top-p cut, one uniform draw from a counter
//      hash of (seed, row).
// Optionally the kept candidates and their probabilities are written out so that tests can compare
// the distribution itself with the host implementation.
// ---------------------------------------------------------------------------
#define SAMPLE_MAX_CAND 1024
#define SAMPLE_THREADS 1024

struct SampleParams {
    float* logits;               // [rows][ld] fp32, modified in place by the repetition penalty
    int ld, n_rows, vocab, vocab_offset;
    float temperature, top_p, rep_penalty;
    int top_k;                   // 0: no top-k (capped at SAMPLE_MAX_CAND candidates)
    const int* past;             // [rows][max_past] token ids (global), may be null
    const int* n_past;           // [rows]
    int max_past;
    int vocab_total;             // tp > 1: size of the whole vocabulary (bounds the merged candidate list); 0: `vocab`
    unsigned long long seed;
    int* out_tokens;             // [rows]
    int* dbg_ids;                // optional [rows][SAMPLE_MAX_CAND]: kept candidates (-1 padded)
    float* dbg_probs;            // optional [rows][SAMPLE_MAX_CAND]
    CommCtx comm;                // tp > 1: `logits` is this rank's vocabulary slice (one row); the ranks exchange
                                 // their candidate lists through symmetric memory and all draw the same token
};

__device__ __forceinline__ unsigned ord_key(float f) {
    unsigned b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long ctr) {
    // splitmix64
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (ctr + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)((z >> 40) + 0.5) * (1.0f / 16777216.0f);
}

// Where candidate (v, id) stands in a list sorted by (value descending, id ascending): the number of
// entries that come before it.
__device__ __forceinline__ int rank_in_list(const float* lv, const int* li, int n, float v, int id) {
    int lo = 0, hi = n;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        const bool before = lv[mid] > v || (lv[mid] == v && li[mid] < id);
        if (before) lo = mid + 1; else hi = mid;
    }
    return lo;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const SampleParams p) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];      // tp > 1: [tp][K] values, [tp][K] ids
    __shared__ float c_val[SAMPLE_MAX_CAND];
    __shared__ int c_id[SAMPLE_MAX_CAND];
    __shared__ float red[32];
    __shared__ int ired[32];
    __shared__ int s_cnt, s_keep;
    __shared__ float s_tot;
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* row = p.logits + (size_t)r * p.ld;
    // ---- 1. repetition penalty
    if (p.past && p.rep_penalty != 1.f) {
        // any number of past tokens, in blocks of the CTA size.  Within a block all values are read before
        // any is written, so a token listed twice in one block is penalised once; the generator passes each
        // distinct past token once, which makes that true across blocks as well.
        const int np = min(p.n_past[r], p.max_past);
        for (int base = 0; base < np; base += SAMPLE_THREADS) {
            const int tok = base + tid < np ? p.past[(size_t)r * p.max_past + base + tid] - p.vocab_offset : -1;
            const bool in = tok >= 0 && tok < p.vocab;
            const float v = in ? row[tok] : 0.f;
            __syncthreads();
            if (in) row[tok] = v > 0.f ? v / p.rep_penalty : v * p.rep_penalty;
            __syncthreads();
        }
    }
    auto block_count = [&](int c) -> int {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        __syncthreads();
        if (lane == 0) ired[warp] = c;
        __syncthreads();
        int t = 0;
#pragma unroll
        for (int w = 0; w < SAMPLE_THREADS / 32; ++w) t += ired[w];
        return t;
    };
    // ---- 2. threshold key: the largest T with count(key >= T) >= K
    const int K = min(p.top_k > 0 ? p.top_k : SAMPLE_MAX_CAND, min(SAMPLE_MAX_CAND, p.vocab));
    unsigned T = 0u;
    for (int bit = 31; bit >= 0; --bit) {
        const unsigned cand = T | (1u << bit);
        int c = 0;
        for (int i = tid; i < p.vocab; i += SAMPLE_THREADS) c += ord_key(row[i]) >= cand;
        if (block_count(c) >= K) T = cand;
    }
    // ---- 3. gather: everything above the threshold, then ties at it until K candidates
    if (tid == 0) s_cnt = 0;
    c_val[tid] = -INFINITY; c_id[tid] = 0x7fffffff;
    __syncthreads();
    for (int i = tid; i < p.vocab; i += SAMPLE_THREADS) {
        const float v = row[i];
        if (ord_key(v) > T) { const int s = atomicAdd(&s_cnt, 1); if (s < SAMPLE_MAX_CAND) { c_val[s] = v; c_id[s] = i; } }
    }
    __syncthreads();
    for (int i0 = 0; i0 < p.vocab; i0 += SAMPLE_THREADS) {        // ties in index order, lowest ids first
        const int i = i0 + tid;
        const bool tie = i < p.vocab && ord_key(row[i]) == T;
        const unsigned m = __ballot_sync(0xffffffffu, tie);
        __syncthreads();
        if (lane == 0) ired[warp] = __popc(m);
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) before += ired[w];
        int total = before;
        for (int w = warp; w < SAMPLE_THREADS / 32; ++w) total += ired[w];
        const int base = s_cnt;
        if (tie) {
            const int s = base + before + __popc(m & ((1u << lane) - 1u));
            if (s < K) { c_val[s] = row[i]; c_id[s] = i; }
        }
        __syncthreads();
        if (tid == 0) s_cnt = min(K, base + total);
        __syncthreads();
        if (s_cnt >= K) break;
    }
    // ---- sort 1024 slots by (value desc, id asc)
    for (int k = 2; k <= SAMPLE_MAX_CAND; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            const int partner = tid ^ j;
            if (partner > tid) {
                const bool up = (tid & k) == 0;
                const float va = c_val[tid], vb = c_val[partner];
                const int ia = c_id[tid], ib = c_id[partner];
                const bool a_first = va > vb || (va == vb && ia < ib);      // a belongs before b
                if (a_first != up) { c_val[tid] = vb; c_val[partner] = va; c_id[tid] = ib; c_id[partner] = ia; }
            }
            __syncthreads();
        }
    int n = min(s_cnt, K);
    // ---- 3b. tensor parallel: every rank holds the K best of its vocabulary slice; the K best overall are
    // among their union.  Each rank publishes its sorted list (values + global ids) in its staging area,
    // the lists are copied into shared memory and merged by rank counting, so that every rank ends up
    // with the same K candidates in the same order and, with the same seed, draws the same token.  No
    // logits are gathered and nothing leaves the device.
    if (p.comm.tp > 1) {
        const CommCtx& c = p.comm;
        __shared__ int s_fail;
        const uint32_t epoch_next = *c.epoch + 1u;
        float* mine = c.part[c.rank] + (size_t)(epoch_next & 1) * c.part_stride;      // [0] count, then K values, K ids
        if (tid == 0) { mine[0] = __int_as_float(n); s_fail = 0; }
        if (tid < K) {
            mine[1 + tid] = c_val[tid];
            mine[1 + K + tid] = __int_as_float(tid < n ? c_id[tid] + p.vocab_offset : 0x7fffffff);
        }
        __threadfence_system();
        __syncthreads();
        if (tid == 0) *c.epoch = epoch_next;
        if (tid < c.tp && tid != c.rank) {
            st_release_sys_u32(c.sig[tid] + c.rank, epoch_next);
            if (!wait_reached(c.sig[c.rank] + tid, epoch_next, c.wait_ns)) {
                report_timeout(c, B2_KID_SAMPLE, tid, epoch_next);
                s_fail = 1;
            }
        }
        __syncthreads();
        float* lv = (float*)dyn_smem;                      // [tp][K]
        int* li = (int*)(lv + (size_t)c.tp * K);           // [tp][K]
        __shared__ int ln[B2_MAX_TP];
        for (int pr = 0; pr < c.tp; ++pr) {
            const float* src = c.part[pr] + (size_t)(epoch_next & 1) * c.part_stride;
            const bool have = pr == c.rank || !s_fail;
            if (tid == 0) ln[pr] = have ? min(K, max(0, __float_as_int(__ldcg(src)))) : 0;
            if (tid < K) {
                lv[pr * K + tid] = have ? __ldcg(src + 1 + tid) : -INFINITY;
                li[pr * K + tid] = have ? __float_as_int(__ldcg(src + 1 + K + tid)) : 0x7fffffff;
            }
        }
        __syncthreads();
        c_val[tid] = -INFINITY; c_id[tid] = 0x7fffffff;
        __syncthreads();
        int total = 0;
        for (int pr = 0; pr < c.tp; ++pr) total += ln[pr];
        // the merged list is as long as the one-rank sampler's would be on the whole vocabulary
        const int vt = p.vocab_total > 0 ? p.vocab_total : p.vocab;
        const int Kg = min(p.top_k > 0 ? p.top_k : SAMPLE_MAX_CAND, min(SAMPLE_MAX_CAND, vt));
        for (int pr = 0; pr < c.tp; ++pr) {
            if (tid < ln[pr]) {
                const float v = lv[pr * K + tid];
                const int id = li[pr * K + tid];
                int pos = tid;                                // entries of its own list that come before it
                for (int q = 0; q < c.tp; ++q)
                    if (q != pr) pos += rank_in_list(lv + q * K, li + q * K, ln[q], v, id);
                if (pos < Kg) { c_val[pos] = v; c_id[pos] = id; }
            }
        }
        __syncthreads();
        n = min(total, Kg);
    }
    const int id_offset = p.comm.tp > 1 ? 0 : p.vocab_offset;      // merged ids are global already
    // ---- 4. softmax, scan, top-p, draw
    const float inv_t = 1.f / fmaxf(p.temperature, 1e-6f);
    const float vmax = c_val[0];
    float e = tid < n ? __expf((c_val[tid] - vmax) * inv_t) : 0.f;
    float x = e;                                                   // inclusive scan of e over the block
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
    if (lane == 31) red[warp] = x;
    __syncthreads();
    if (warp == 0) {
        float w = red[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const float y = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w += y; }
        red[lane] = w;
    }
    __syncthreads();
    const float cum = x + (warp ? red[warp - 1] : 0.f);
    if (tid == SAMPLE_THREADS - 1) s_tot = cum;
    if (tid == 0) s_keep = n;
    __syncthreads();
    const float tot = s_tot;
    // keep = 1 + number of candidates whose cumulative mass is still below top_p
    if (p.top_p < 1.f && tid < n && cum / tot >= p.top_p) atomicMin(&s_keep, tid + 1);
    __syncthreads();
    const int keep = s_keep;
    if (tid == keep - 1) s_tot = cum;                              // mass of the kept prefix
    __syncthreads();
    const float kept = s_tot;
    const float u = uniform01(p.seed, (unsigned long long)r) * kept;
    if (tid == 0) s_cnt = keep - 1;                                // default: last kept (guards rounding)
    __syncthreads();
    if (tid < keep && cum >= u) atomicMin(&s_cnt, tid);
    __syncthreads();
    if (tid == 0) p.out_tokens[r] = c_id[s_cnt] + id_offset;
    if (p.dbg_ids) {
        p.dbg_ids[(size_t)r * SAMPLE_MAX_CAND + tid] = tid < keep ? c_id[tid] + id_offset : -1;
        p.dbg_probs[(size_t)r * SAMPLE_MAX_CAND + tid] = tid < keep ? e / kept : 0.f;
    }
}

B2_API int b2_sample(const SampleParams* p, cudaStream_t s) {
    if (p->n_rows < 1 || p->vocab < 1 || p->temperature <= 0.f || p->top_k < 0 || p->top_p <= 0.f) return cudaErrorInvalidValue;
    size_t smem = 0;
    if (p->comm.tp > 1) {
        // one row per launch under tensor parallelism (the exchange is the launch's only CTA's)
        const int K = p->top_k > 0 && p->top_k < SAMPLE_MAX_CAND ? p->top_k : SAMPLE_MAX_CAND;
        if (p->n_rows != 1 || p->comm.part_stride < 1 + 2 * K) return cudaErrorInvalidValue;
        smem = (size_t)p->comm.tp * K * 8;
        static SmemOptIn optin;
        cudaError_t e = optin.ensure(sample_kernel, smem + 16 * 1024);
        if (e != cudaSuccess) return e;
    }
    sample_kernel<<<p->n_rows, SAMPLE_THREADS, smem, s>>>(*p);
    return cudaGetLastError();
}
B2_API int b2_sizeof_sample_params() { return (int)sizeof(SampleParams); }
