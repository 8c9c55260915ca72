// INT8-activation linear layers: dynamic per-row activation quantisation, and
// W8A8 / W4A8 matrix products on the int8 tensor-core path (m16n8k32, s32 accumulate).
//
// The reference keeps these as an optional path beside its w4a16 kernels
// (reference: src/kernels/activation_quant.hip, src/kernels/gemv_w8a8.hip,
// src/kernels/gemv_w4a8.hip, src/kernels/gemm_w8a8.hip; conversion in
// src/model/weight_loader.py:122-249).  Here one kernel serves one row (GEMV) up to
// many rows (GEMM): the weight rows are the 16-row A operand, eight activation rows
// are the B operand, so a single token already fills a whole instruction.
//
// Layouts
//   W8:  int8  [N][K]   per-output-channel scale fp32 [N]
//   W4:  int32 [N][K/8] signed nibbles (nibble b of word c = column 8c+b, zero point
//        already subtracted), per-group scale fp16 [K/group][N]
//   x:   int8  [T][K]   per-row scale fp32 [T]
// out[t][n] = x_scale[t] * sum_k xq[t][k] * w[n][k] * (w_scale[n] | g_scale[k/group][n])
//
// The k order inside an instruction is free as long as both operands agree, so every
// lane fetches 16 contiguous bytes of its weight row and of its activation row and
// feeds them to two instructions; no shared-memory staging is needed.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.cuh"

namespace {

constexpr int Q8_WARPS = 8;
constexpr int Q8_THREADS = Q8_WARPS * 32;

__device__ __forceinline__ void mma_s8(int (&d)[4], int a0, int a1, int a2, int a3, int b0, int b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ int4 ldg16(const void* p) { return __ldg(reinterpret_cast<const int4*>(p)); }

// eight signed nibbles -> (even columns, odd columns) as packed int8
__device__ __forceinline__ void nib8(int w, int& even, int& odd) {
    const unsigned lo = (unsigned)w & 0x0F0F0F0Fu, hi = ((unsigned)w >> 4) & 0x0F0F0F0Fu;
    even = (int)__vsub4(lo ^ 0x08080808u, 0x08080808u);
    odd = (int)__vsub4(hi ^ 0x08080808u, 0x08080808u);
}

// One CTA: 16 output channels x (8*NT) activation rows; its warps split K.
template <int NT, bool W4>
__global__ void __launch_bounds__(Q8_THREADS) q8_linear_kernel(Quant8Params p) {
    __shared__ float red[Q8_WARPS][NT][32][4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16, tb = blockIdx.y * (8 * NT);
    const int ra = min(n0 + g, p.N - 1), rb = min(n0 + g + 8, p.N - 1);      // clamped; masked at the store
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;

    const int8_t* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int tok = tb + 8 * j + g;
        xok[j] = tok < p.T;
        xrow[j] = p.xq + (size_t)min(tok, p.T - 1) * p.K;
    }

    if constexpr (!W4) {
        const int8_t* wa = reinterpret_cast<const int8_t*>(p.w) + (size_t)ra * p.K + 16 * t;
        const int8_t* wb = reinterpret_cast<const int8_t*>(p.w) + (size_t)rb * p.K + 16 * t;
        int iacc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) iacc[j][c] = 0;
#pragma unroll 2
        for (int k0 = warp * 64; k0 < p.K; k0 += Q8_WARPS * 64) {
            const int4 a = ldg16(wa + k0), b = ldg16(wb + k0);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                int4 x = make_int4(0, 0, 0, 0);
                if (xok[j]) x = ldg16(xrow[j] + k0 + 16 * t);
                mma_s8(iacc[j], a.x, b.x, a.y, b.y, x.x, x.y);
                mma_s8(iacc[j], a.z, b.z, a.w, b.w, x.z, x.w);
            }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[j][c] = (float)iacc[j][c];
    } else {
        const int* wa = reinterpret_cast<const int*>(p.w) + (size_t)ra * (p.K >> 3) + 4 * t;
        const int* wb = reinterpret_cast<const int*>(p.w) + (size_t)rb * (p.K >> 3) + 4 * t;
        const int per = p.group >> 7;                                        // 128-column blocks per scale group
        for (int kb = warp; kb * 128 < p.K; kb += Q8_WARPS) {
            const int4 a = ldg16(wa + kb * 16), b = ldg16(wb + kb * 16);
            const int grp = kb / per;
            const float sa = __half2float(__ldg(p.g_scale + (size_t)grp * p.N + ra));
            const float sb = __half2float(__ldg(p.g_scale + (size_t)grp * p.N + rb));
            int ae[4], ao[4], be[4], bo[4];
            nib8(a.x, ae[0], ao[0]); nib8(a.y, ae[1], ao[1]); nib8(a.z, ae[2], ao[2]); nib8(a.w, ae[3], ao[3]);
            nib8(b.x, be[0], bo[0]); nib8(b.y, be[1], bo[1]); nib8(b.z, be[2], bo[2]); nib8(b.w, be[3], bo[3]);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                int4 x0 = make_int4(0, 0, 0, 0), x1 = x0;
                if (xok[j]) {
                    x0 = ldg16(xrow[j] + kb * 128 + 32 * t);
                    x1 = ldg16(xrow[j] + kb * 128 + 32 * t + 16);
                }
                const int xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                int d[4] = {0, 0, 0, 0};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int xe = (int)__byte_perm((unsigned)xw[2 * i], (unsigned)xw[2 * i + 1], 0x6420);
                    const int xo = (int)__byte_perm((unsigned)xw[2 * i], (unsigned)xw[2 * i + 1], 0x7531);
                    mma_s8(d, ae[i], be[i], ao[i], bo[i], xe, xo);
                }
                acc[j][0] += (float)d[0] * sa; acc[j][1] += (float)d[1] * sa;
                acc[j][2] += (float)d[2] * sb; acc[j][3] += (float)d[3] * sb;
            }
        }
    }

#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) red[warp][j][lane][c] = acc[j][c];
    __syncthreads();
    for (int idx = threadIdx.x; idx < NT * 128; idx += Q8_THREADS) {
        const int j = idx >> 7, l = (idx >> 2) & 31, c = idx & 3;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < Q8_WARPS; ++w) s += red[w][j][l][c];
        const int n = n0 + (l >> 2) + ((c & 2) ? 8 : 0);
        const int tok = tb + 8 * j + 2 * (l & 3) + (c & 1);
        if (n < p.N && tok < p.T) {
            float v = s * __ldg(p.x_scale + tok);
            if constexpr (!W4) v *= __ldg(p.w_scale + n);
            if (p.out_f16) reinterpret_cast<__half*>(p.out)[(size_t)tok * p.ldo + n] = __float2half(v);
            else reinterpret_cast<float*>(p.out)[(size_t)tok * p.ldo + n] = v;
        }
    }
}

// One CTA per activation row: scale = max|x| / 127, xq = round-to-nearest-even(x / scale).
__global__ void __launch_bounds__(256) act_quant_kernel(ActQuantParams p) {
    __shared__ float s_max[8];
    const int r = blockIdx.x;
    const __half2* x = reinterpret_cast<const __half2*>(p.x + (size_t)r * p.ldx);
    float m = 0.f;
    for (int i = threadIdx.x; i < (p.K >> 1); i += blockDim.x) {
        const float2 v = __half22float2(x[i]);
        m = fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y)));
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = m;
    __syncthreads();
    m = s_max[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, s_max[w]);
    const float scale = __fdiv_rn(fmaxf(m, 1e-12f), 127.f);
    if (threadIdx.x == 0) p.scale[r] = scale;
    char2* q = reinterpret_cast<char2*>(p.xq + (size_t)r * p.K);
    for (int i = threadIdx.x; i < (p.K >> 1); i += blockDim.x) {
        const float2 v = __half22float2(x[i]);
        const int a = max(-128, min(127, __float2int_rn(__fdiv_rn(v.x, scale))));
        const int b = max(-128, min(127, __float2int_rn(__fdiv_rn(v.y, scale))));
        q[i] = make_char2((signed char)a, (signed char)b);
    }
}

template <bool W4>
int launch_q8(const Quant8Params& p, cudaStream_t s) {
    const int nb = (p.N + 15) / 16;
    if (p.T <= 8) q8_linear_kernel<1, W4><<<dim3(nb, 1), Q8_THREADS, 0, s>>>(p);
    else if (p.T <= 16) q8_linear_kernel<2, W4><<<dim3(nb, 1), Q8_THREADS, 0, s>>>(p);
    else if (p.T <= 32) q8_linear_kernel<4, W4><<<dim3(nb, 1), Q8_THREADS, 0, s>>>(p);
    else q8_linear_kernel<8, W4><<<dim3(nb, (p.T + 63) / 64), Q8_THREADS, 0, s>>>(p);
    return cudaGetLastError();
}

}  // namespace

B2_API int b2_linear_q8(const Quant8Params* p, cudaStream_t s) {
    if (p->T < 1 || p->N < 1 || p->K < 1 || p->ldo < p->N) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(p->w) | reinterpret_cast<uintptr_t>(p->xq)) & 15) return cudaErrorInvalidValue;
    if (p->w4) {
        if (p->K % 128 || p->group < 128 || p->group % 128 || p->K % p->group || !p->g_scale) return cudaErrorInvalidValue;
        return launch_q8<true>(*p, s);
    }
    if (p->K % 64 || !p->w_scale) return cudaErrorInvalidValue;
    return launch_q8<false>(*p, s);
}

B2_API int b2_act_quant(const ActQuantParams* p, cudaStream_t s) {
    if (p->T < 1 || p->K < 2 || (p->K & 1) || (p->ldx & 1)) return cudaErrorInvalidValue;
    act_quant_kernel<<<p->T, 256, 0, s>>>(*p);
    return cudaGetLastError();
}

B2_API int b2_sizeof_quant8_params() { return (int)sizeof(Quant8Params); }
B2_API int b2_sizeof_act_quant_params() { return (int)sizeof(ActQuantParams); }
