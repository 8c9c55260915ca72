// Parameter blocks of the persistent projection-chain kernel (csrc/chain.cu).
#pragma once
#include "gemv.cuh"

#define CH_MAX_OPS 4
#ifndef CH_WARPS
#define CH_WARPS 8
#endif
#define CH_THREADS (CH_WARPS * 32)
#define CH_MAX_STAGES 8
#ifndef CH_MIN_STAGES
#define CH_MIN_STAGES 2
#endif
#define CH_STAGE_BYTES 5120          // two k64-blocks of one 64-column warp tile + scale/zero pairs of up to four groups
#define CH_SMEM_LIMIT (227 * 1024)

// One INT4 projection of a chain.  Weight layout and epilogues are those of the
// stand-alone GEMV (gemv.cuh); the output tile of the epilogues is 64 columns.
struct ChainOp {
    const uint4* qfrag;       // [NWT][KB][4][32] fragment-ordered nibbles (2 KB per k64-block of a warp tile)
    const uint2* szfrag;      // [NWT*4][G][8]
    const __half* x;          // [rows][ldx] fp16 input, or null: the lazily normalised residual stream `ln`
    int ldx, K, KB, NWT, G, off32, gshift;
    // work split, set by the launcher: granules of gsz k64-blocks, cBase (+1 for the first cRem CTAs) per CTA
    int gsz, cBase, cRem;
    int pmax;                 // upper bound of split-K pieces per warp tile (set by the launcher)
    int pad;
    LazyNorm ln;
    GemvEpi epi;              // epi.ss_np: row stride of ss_part; a FINISH tile writes entry n0/64
};

struct ChainParams {
    int n_ops, rows;
    int stages;               // weight-ring depth per warp (set by the launcher)
    int cstride;              // ints per op in `counters`
    ChainOp op[CH_MAX_OPS];
    float* scratch;           // split-K pieces: [warp tile][piece][row][64]
    int* counters;            // [CH_MAX_OPS][cstride] tile arrivals, then done[CH_MAX_OPS], then exit; zero between launches
    long long* prof;          // optional [grid * CH_WARPS][CH_MAX_OPS][8] per-warp timing record (null: off)
    CommCtx comm;
};

B2_API int b2_chain(const ChainParams* p, cudaStream_t stream);
B2_API int b2_chain_feasible(const ChainParams* p);
B2_API long long b2_chain_scratch_floats(int KB, int NWT, int rows);
