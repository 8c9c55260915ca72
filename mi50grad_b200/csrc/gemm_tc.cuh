// Parameters of the tcgen05 INT4 GEMM (csrc/gemm_tc.cu).
#pragma once
#include "common.cuh"

#define TC_EPI_STORE_F16 0
#define TC_EPI_SILU_PAIR 1
#define TC_EPI_STORE_F32 2
#define TC_EPI_RESID_F32 3       // out32[t][n] += y

struct GemmTcParams {
    const uint4* qfrag;      // [NTL/4][KB][4][32] packed nibbles
    const uint2* szfrag;     // [NTL][G][8]
    int K, KB, NTL, G, off32, gshift;
    int T;                   // token rows in this launch's activation matrix
    int t_tile;              // tokens per CTA (multiple of 16, <= 512)
    int n_valid, ldo, epi, stages;
    void* out;
    int* status;             // [0] set to 1 when a bounded wait expired
    int pad;
    int dense;               // set by the launcher: weights are fp16 and come through a tensor map
};


B2_API int b2_gemm_int4_tc(const GemmTcParams* p, const void* x, int ldx, cudaStream_t stream);
B2_API int b2_gemm_f16_tc(const GemmTcParams* p, const void* w, int ldw, const void* x, int ldx, cudaStream_t stream);
