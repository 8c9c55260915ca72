// Parameter blocks of the decode-path GEMV kernels (shared with the step driver).
#pragma once
#include "common.cuh"

// Epilogue modes: what happens to a finished [rows x 128] output tile.
#define EPI_STORE_F16 0      // out16[row][n]  = y
#define EPI_SILU_PAIR 1      // out16[row][j]  = silu(y[gate_j]) * y[up_j]  (gate/up interleaved by 8)
#define EPI_STORE_F32 2      // out32[row][n]  = y
#define EPI_FINISH    3      // row-parallel: all-reduce + residual add + next RMSNorm

// Flags of EPI_FINISH.
#define FIN_NO_COMM     1    // keep the sum local (tp == 1, or a deferred attention partial)
#define FIN_NO_H_WRITE  2    // do not update the residual stream (deferred_consistent attention)
#define FIN_SAVE_EXTRA  4    // save this rank's partial into `extra`
#define FIN_ADD_EXTRA   8    // add `extra` to the partial before it is exchanged
#define FIN_NO_NORM     16   // skip the RMSNorm (xn not written)
#define FIN_TEST_WITHHOLD_SIGNAL 32  // test hook: do not signal peers, so the bounded wait runs out

// "Lazy" RMSNorm input: instead of a materialised fp16 vector a consumer kernel can be
// given the fp32 residual stream, the per-tile sums of squares its producer left behind
// and the norm weights; it then forms x[k] = h[k] * rsqrt(sum(ss)/H + eps) * w[k] while
// staging its activations.  This removes the serial normalise-and-store tail between a
// row-parallel projection and its consumer.
struct LazyNorm {
    const float* h;          // [rows][H] residual stream (null: use the fp16 x instead)
    const float* ss;         // [rows][np] partial sums of squares
    const __half* w;         // [H]
    int np, H;
    float eps;
    int pad;
};

__device__ __forceinline__ float lazy_inv_rms(const LazyNorm& ln, int row, int lane) {
    // one warp: sum the partials in a fixed order
    // (the first four loads of a lane are requested together; the order of the additions is unchanged)
    float s = 0.f, v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = (lane + 32 * u < ln.np) ? ln.ss[(size_t)row * ln.np + lane + 32 * u] : 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) s += v[u];
    for (int i = lane + 128; i < ln.np; i += 32) s += ln.ss[(size_t)row * ln.np + i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    return rsqrtf(s / (float)ln.H + ln.eps);
}

struct GemvEpi {
    int mode;
    int ldo;                 // row stride of out (elements)
    int n_valid;             // real number of outputs (columns beyond are padding)
    int fin_flags;
    void* out;               // f16 / f32 output for the STORE / SILU modes
    float* h;                // [rows][n_valid] fp32 residual stream (FINISH)
    const __half* norm_w;    // [n_valid] multiplier of the following RMSNorm
    __half* xn;              // [rows][n_valid] normalised output
    float* extra;            // [rows][n_valid] saved / added partial
    float* local_part;       // unused (kept for layout stability)
    float* hout;             // [rows][n_valid] where h + sum is written (h itself, or a scratch row
                             // buffer when FIN_NO_H_WRITE)
    float* ss_part;          // [rows][ceil(n_valid/128)] per-tile sums of squares of hout
    float eps;
    int ss_np;               // row stride of ss_part (0: one entry per 128-column tile).  When it is a multiple
                             // of that, a 128-column tile writes its sum into the first of its entries and
                             // zero into the others, so that producers with 64-column tiles can share the buffer
};

struct GemvInt4Params {
    const uint4* qfrag;      // [NTL][KB][32] fragment-ordered nibbles
    const uint2* szfrag;     // [NTL/4][G][4][8] (scale_lo, scale_hi, zero_lo, zero_hi) halves
    const __half* x;         // [rows][ldx]
    int ldx, rows, K, KB, NTL, G;
    int off32, gshift;       // group of chunk c = (c + off32) >> gshift   (chunk = 32 k)
    int k_splits, L;         // CTAs along K, k64-blocks per warp
    int cluster_splitk;      // set by the launcher: the k_splits CTAs of an output tile form a thread-block cluster
                             // and reduce their partial tiles through distributed shared memory
    int tag_base;            // see tag_word
    float* scratch;          // [k_splits][rows][NTL*16] split-K partials
    int* counters;           // [gridDim.x + 1], zero between launches
    // Tagged split-K hand-off (optional): with tag_word set, the partners of an output tile store their
    // partial sums as {value, tag} pairs (tag = *tag_word + tag_base, never 0 and never repeated on this
    // scratch buffer while an older pair can still sit in it) and the CTA of slice 0 polls them: no fence, no
    // counter, no second trip to L2.  scratch then holds (k_splits - 1) x rows x N such pairs.  The caller
    // must keep the whole grid resident (the launcher checks and falls back to the counter protocol).
    const unsigned int* tag_word;
    // L2 prefetch for the INT4 GEMV that follows in the stream (optional, pf_q != null): when a warp has
    // requested the last of its own weights it asks L2 for the first pf_blocks k-blocks of "its" warps of the
    // next launch (grid pf_nx x pf_ks, pf_L blocks per warp, pf_KB blocks per tile), so that HBM keeps
    // streaming through this kernel's reduction tail and the next kernel's start.
    const uint4* pf_q;
    int pf_KB, pf_L, pf_nx, pf_ks, pf_blocks, pf_pad;
    // ... or (pf_span != null) for pf_span_bytes of anything else the next kernel reads first, e.g. the DeltaNet state
    const void* pf_span;
    long long pf_span_bytes;
    LazyNorm ln;
    GemvEpi epi;
    CommCtx comm;
};

struct GemvF16Params {
    const __half* w;         // [N][ldw] row-major (out_features x in_features)
    const __half* x;         // [rows][ldx]
    int ldw, ldx, rows, K, N;
    int k_splits, kslice;    // kslice: multiple of 256
    float* scratch;
    int* counters;
    LazyNorm ln;
    GemvEpi epi;
    CommCtx comm;
};
