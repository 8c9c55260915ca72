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
