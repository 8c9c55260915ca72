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
    // Hand-off between the projections of one launch, wired by the launcher: a producer's epilogue
    // also stores {value, tag} pairs (one 8-byte store each), and its consumer polls those instead of
    // waiting for a counter: the data is its own arrival flag, nothing is fenced or counted.
    float2* th_out; float2* tss_out; uint2* tact_out;                  // this op's tagged outputs (null: none)
    const float2* th_in; const float2* tss_in; const uint2* tact_in;   // tagged input replacing ln.h + ln.ss / x
    const float2* th_res;     // FINISH: tagged residual stream written by op `res_op` of this launch (null: epi.h)
    int in_op, res_op;
};

struct ChainParams {
    int n_ops, rows;
    int stages;               // weight-ring depth per warp (set by the launcher)
    int xf_chunks;            // widest activation window any CTA stages, in 32-k chunks (set by the launcher)
    ChainOp op[CH_MAX_OPS];
    float2* scratch;          // partial tiles that cross CTAs, {value, tag}: [warp tile][piece][row][64]
    unsigned int* counters;   // [0] CTAs that have left (zero between launches), [1] launch generation (never reset)
    float2* tag_h;            // [rows][tag_h_cols]   tagged residual stream
    float2* tag_ss;           // [rows][tag_ss_cols]  tagged per-tile sums of squares
    uint2* tag_act;           // [rows][tag_act_cols] tagged fp16 pairs of the SiLU output
    int tag_h_cols, tag_ss_cols, tag_act_cols, pad1;
    long long* prof;          // optional [grid * CH_WARPS][CH_MAX_OPS][8] per-warp timing record (null: off)
    CommCtx comm;
};

B2_API int b2_chain(const ChainParams* p, cudaStream_t stream);
B2_API int b2_chain_feasible(const ChainParams* p);
B2_API long long b2_chain_scratch_floats(int KB, int NWT, int rows);
