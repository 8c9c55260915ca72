// Parameter blocks and host launchers of every kernel in this library.
#pragma once
#include "gemv.cuh"

struct AttnParams {
    const __half* q;         // [rows][ldq]: Q heads at column h*hd, gates at gate_off + h*hd
    int ldq, gate_off;       // gate_off < 0: no output gate
    const __half* kcache;    // [seq][max_seq][nkv][hd]
    const __half* vcache;
    const RowMeta* rows;
    __half* out;             // [rows][ldo], head h at column h*hd
    int ldo, n_rows, nq, nkv, max_seq, splits;
    float scale;
    float* scratch;          // [rows][nkv][splits][G][hd+2]
    int* counters;           // [rows*nkv], zero between launches
};

struct DeltaParams {
    const __half* proj;      // [rows][ld] in-projection outputs
    int ld, off_q, off_k, off_v, off_z, off_a, off_b;   // off_a < 0: compute a,b here
    const __half* xn;        // [rows][ldx] normalised layer input (for in-kernel a,b)
    int ldx, H;
    const __half* wa;        // [nv][H]
    const __half* wb;        // [nv][H]
    const __half* conv_w;    // [2*nk*dk + nv*dv][4], channel order q | k | v
    __half* conv_state;      // [seq][nv][dv/32][2*dk+32][3] private histories (oldest first)
    float* state;            // [seq][nv][dk][dv]
    const float* A_log;      // [nv]
    const __half* dt_bias;   // [nv]
    const __half* norm_w;    // [dv]
    const int* seq_rows;     // [n_seqs+1] row range of each launched sequence
    const RowMeta* rows;     // rows[seq_rows[i]].seq = state slot of launched sequence i
    __half* out;             // [rows][ldo], head j at column j*dv
    int ldo, nk, nv, n_seqs;
    float eps;
    int commit;              // 0: leave state and conv history untouched (dry run for tree verification)
    LazyNorm ln;             // if ln.h: the a/b projections read the lazily normalised residual stream
};

struct ArgmaxParams {
    const float* logits;     // [rows][ld] this rank's vocabulary slice
    int ld, n_rows, vocab_local, vocab_offset;
    int blocks;              // CTAs per row
    float* scratch;          // [rows][blocks][2]
    int* counters;           // [rows]
    int* out_tokens;         // [rows]
    SeqState* seqs;          // if non-null: seqs[rows[r].seq].token = token of row r
    const RowMeta* rows;
    CommCtx comm;
};

struct CollParams {
    CommCtx comm;
    const float* in;         // local input [n] fp32 (may be null when in16 is given)
    const __half* in16;      // local input [n] fp16
    float* out;              // local output [n]: out = sum (+ out if residual)
    __half* out16;           // optional fp16 copy of the result
    float* gather[B2_MAX_TP];// two-shot: per-rank symmetric result buffers [n]
    float* mc_gather;        // multicast mapping of gather (or null)
    size_t n;                // elements, multiple of 4
    int residual;            // 1: out += sum
    int twoshot;
    int* counters;           // [4] local, zero between launches
    int test_withhold;       // test hook: never signal, so that the bounded wait expires
    int pushed;              // 1: the producers already stored every rank's slice contributions into the owners'
                             //    staging buffers ([source rank][slice]); nothing to publish, reduce from local memory
};

// Sequence-parallel hand-off after a row-parallel many-row projection (csrc/comm.cu, rs_norm_ag_kernel):
// reduce-scatter by token rows, residual add and RMSNorm on this rank's rows, all-gather of the fp16 result
// straight into every rank's activation buffer, where the next GEMM's TMA loads find it.
struct SeqParParams {
    CommCtx comm;
    float* h;                    // local residual stream [T][H] fp32: only this rank's rows are read and updated
    const __half* norm_w;        // weights of the RMSNorm that follows
    __half* xn[B2_MAX_TP];       // every rank's activation buffer [T][H] fp16 (symmetric memory)
    __half* mc_xn;               // multicast mapping of that buffer (or null: plain peer stores)
    float* hlast[B2_MAX_TP];     // every rank's slot [H] for the fp32 residual of row T-1
    int T, H, rows_per;          // rank r owns rows [r * rows_per, min(T, (r + 1) * rows_per))
    float eps;
    int* counters;               // [4] local, zero between launches
    int test_withhold;           // test hook: never signal, so that the bounded wait expires
    int pad;
};

// ---- speculative verification (csrc/speculative.cu)
#define SPEC_MAX_NODES 16          // rows per sequence in one verify step: the pending token + up to 15 drafts

// What the DeltaNet verify kernel leaves behind for the commit kernel, one block per
// (linear-attention layer, launched sequence): normalised keys, the rank-1 update vectors
// u, the cumulative log-decay G along each node's path, and the raw conv inputs.
struct SpecStage {
    unsigned char* base;
    long long layer_stride, seq_stride;      // bytes
    int off_k;                               // f32 [SPEC_MAX_NODES][nk][dk]
    int off_u;                               // f32 [SPEC_MAX_NODES][nv][dv]
    int off_g;                               // f32 [SPEC_MAX_NODES][nv]
    int off_x;                               // f16 [SPEC_MAX_NODES][2*nk*dk + nv*dv]
};

struct SpecAcceptParams {
    const int* out_tokens;       // [rows] the model's greedy prediction after each row
    const int* row_tokens;       // [rows] tokens that were fed (-1: the sequence's pending token)
    const RowMeta* rows;
    const int* seq_rows;         // [n_seqs+1]
    SeqState* seqs;              // len += accepted path length, token = next pending token
    int* acc;                    // [n_seqs][SPEC_MAX_NODES+2]: path length, slot of the root, path node indices
    int* result;                 // [n_seqs][SPEC_MAX_NODES+2]: accepted drafts, next token, accepted draft tokens
    int n_seqs, pad;
};

struct DeltaCommitParams {
    float* state0;               // state of the first linear-attention layer [seq][nv][dk][dv]
    __half* conv0;               // conv history of the first linear-attention layer
    long long state_layer_stride, conv_layer_stride;   // elements
    SpecStage st;
    const int* acc;
    const RowMeta* rows;
    const int* seq_rows;
    int nk, nv, n_seqs, n_layers;
};

struct KvCompactParams {
    __half* k0; __half* v0;      // caches of the first full-attention layer [seq][max_seq][nkv][hd]
    long long layer_stride;      // elements
    const int* acc;
    const RowMeta* rows;
    const int* seq_rows;
    int n_layers, n_seqs, nkv, hd, max_seq, pad;
};

B2_API int b2_deltanet_verify(const DeltaParams* p, const SpecStage* st, int layer, int dk, int dv, cudaStream_t s);
B2_API int b2_deltanet_commit(const DeltaCommitParams* p, int dk, int dv, cudaStream_t s);
B2_API int b2_spec_accept(const SpecAcceptParams* p, cudaStream_t s);
B2_API int b2_kv_compact(const KvCompactParams* p, cudaStream_t s);
B2_API int b2_allreduce(const CollParams* p, int max_ctas, cudaStream_t s);
B2_API int b2_rs_norm_ag(const SeqParParams* p, cudaStream_t s);
B2_API int b2_gemv_int4(const GemvInt4Params* p, cudaStream_t stream);
B2_API int b2_gemv_f16(const GemvF16Params* p, cudaStream_t stream);
B2_API int b2_decode_attn(const AttnParams* p, int hd, cudaStream_t s);
B2_API int b2_attn_rows(const AttnParams* p, const int* seq_rows, int n_seqs, int hd, cudaStream_t s);
B2_API int b2_attn_prefill_tc(const AttnParams* p, int row_base, int n_rows_seq, int n_slots, int hd, int* status,
                              cudaStream_t s);
B2_API int b2_deltanet_step(const DeltaParams* p, int dk, int dv, cudaStream_t s);
B2_API int b2_deltanet_chunk(const DeltaParams* p, const void* ab, int ld_ab, void* qk_scratch, int ld_qk, int n_rows,
                             void* tw_scratch, int dk, int dv, cudaStream_t s);
B2_API long long b2_deltanet_tw_floats(int nv, int n_rows);
B2_API int b2_ab_proj(const void* x, int ldx, const void* wa, const void* wb, int nv, int H, void* ab, int ld_ab,
                      int rows, cudaStream_t s);
B2_API int b2_argmax(const ArgmaxParams* p, cudaStream_t s);
B2_API int b2_prepare_rows(const void* tmpl, const void* seqs, void* rows, int n, unsigned int* step_word, cudaStream_t s);
B2_API int b2_advance(void* seqs, const int* add, int n, int add_const, cudaStream_t s);
B2_API int b2_embed_rmsnorm(const void* embed, const int* row_tokens, const void* rows, const void* seqs,
                            const void* w, float* h, void* xn, float* ss_part, int np, int n_rows, int H,
                            float eps, int vocab, cudaStream_t s);
B2_API int b2_load_rmsnorm(const void* emb16, const float* emb32, const void* w, float* h, void* xn,
                           float* ss_part, int np, int n_rows, int H, float eps, cudaStream_t s);
B2_API int b2_add_rmsnorm(float* h, const float* delta32, const void* delta16, const void* w, void* xn,
                          float* xn32, int n_rows, int H, float eps, cudaStream_t s);
B2_API int b2_qknorm_rope_cachew(void* qkv, int ld, const void* rows, const void* q_norm, const void* k_norm,
                                 const float* cos_tab, const float* sin_tab, void* kcache, void* vcache,
                                 int n_rows, int nq, int nkv, int hd, int rot, int max_seq, int interleaved,
                                 float eps, cudaStream_t s);

// ---- INT8-activation products (csrc/quant8.cu) as the step driver uses them
struct Quant8Params {
    const void* w;
    const float* w_scale;
    const __half* g_scale;
    const int8_t* xq;
    const float* x_scale;
    void* out;
    int K, N, T, ldo, group, out_f16, w4, pad;
};
struct ActQuantParams {
    const __half* x;
    int8_t* xq;
    float* scale;
    int T, K, ldx, pad;
};
B2_API int b2_linear_q8(const Quant8Params* p, cudaStream_t s);
B2_API int b2_act_quant(const ActQuantParams* p, cudaStream_t s);
B2_API int b2_silu_mul(const void* gate, const void* up, void* out, size_t n, cudaStream_t s);
B2_API int b2_residual_add(float* h, const float* d32, const void* d16, size_t n, cudaStream_t s);
B2_API int b2_residual_add_ss(float* h, const float* d32, float* ss, int np, int n_rows, int H, cudaStream_t s);
