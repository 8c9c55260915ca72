// Parameters of the tcgen05 INT4 GEMM (csrc/gemm_tc.cu).
#pragma once
#include "common.cuh"

#define TC_EPI_STORE_F16 0
#define TC_EPI_SILU_PAIR 1
#define TC_EPI_STORE_F32 2
#define TC_EPI_RESID_F32 3       // out32[t][n] += y
#define TC_EPI_PUSH_F32 4        // tensor parallel: y goes straight into the symmetric staging buffer of the
                                 // rank that will reduce that slice of the [T x n_valid] output (reduce-scatter
                                 // fused into the GEMM epilogue; the collective kernel then reads local memory only)

struct GemmTcParams {
    const uint4* qfrag;      // [NTL/4][KB][4][32] packed nibbles
    const uint2* szfrag;     // [NTL/4][G][4][8]
    int K, KB, NTL, G, off32, gshift;
    int T;                   // token rows in this launch's activation matrix
    int t_tile;              // tokens per CTA (multiple of 16, <= 512)
    int n_valid, ldo, epi, stages;
    void* out;
    int* status;             // [0] set to 1 when a bounded wait expired
    int m_halves;            // 2: CTAs own 256 outputs (two accumulators sharing each activation tile; t_tile <= 256,
                             // N a multiple of 256); else 128 outputs
    int dense;               // set by the launcher: weights are fp16 and come through a tensor map
    // TC_EPI_PUSH_F32: the flattened output (float4 units) is cut into push_tp slices of push_per; slice o
    // lives on rank o at push[o] + parity offset + (push_rank * push_per + index in slice) * 4 floats
    float* push[B2_MAX_TP];
    const unsigned int* epoch;   // collective epoch counter of this rank (parity of the next collective)
    long long part_stride;       // floats between the two parity halves of a staging buffer
    int push_tp, push_rank;
    unsigned int push_per;       // float4 elements per slice
    int k_splits;                // TC_EPI_RESID_F32 only: CTAs along K per output tile (grid z); their partial
                                 // products are added to out with atomic adds (0 or 1: no split)
    int cta_pair;                // 1: adjacent output tiles run as CTA pairs (cta_group::2 MMAs, M = 256 over two SMs); needs
                                 // 128-output CTAs, t_tile 256 or 512 dividing T, an even number of output tiles
    int pad3;
};


B2_API int b2_gemm_int4_tc(const GemmTcParams* p, const void* x, int ldx, cudaStream_t stream);
B2_API int b2_gemm_f16_tc(const GemmTcParams* p, const void* w, int ldw, const void* x, int ldx, cudaStream_t stream);
