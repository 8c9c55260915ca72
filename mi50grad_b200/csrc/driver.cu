// Decode step driver: owns the per-token launch sequence of one rank and its
// CUDA-graph capture/replay.
//
// It is the counterpart of the reference's C dispatch loops (reference:
// src/runtime/c_dispatch.c:975-1213, c_dispatch_v2.c:501, c_graph_dispatch.c:458-540):
// Python flattens the model into plain structs once, then one C call issues a
// whole token.  What is different on purpose:
//  * one process drives one GPU, so there is no device switching and no
//    host-side event choreography between GPUs: cross-GPU ordering lives inside
//    the kernels (flags in symmetric memory);
//  * nothing is patched between tokens.  Positions, cache slots and the input
//    token live in device memory (SeqState / RowMeta), so the whole step,
//    embedding gather to arg-max, is ONE graph that is replayed unchanged (the
//    reference re-writes kernel-node parameters of 2 graphs per layer per token:
//    c_graph_dispatch.c:389-431);
//  * a replay loop can run any number of tokens without returning to the host.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include "kernels.cuh"
#include "gemm_tc.cuh"
#include "chain.cuh"

#define LIN_INT4 0
#define LIN_F16 1
#define LIN_NONE 2

struct LinearDesc {
    int kind;
    int K, N;                     // logical in/out features (N: valid outputs)
    int KB, NTL, G, off32, gshift;
    int k_splits, L;              // int4 launch shape
    int ldw, kslice;              // f16 launch shape
    int pad;
    const void* w;                // qfrag or fp16 weights
    const void* sz;               // szfrag
};

struct LayerDesc {
    int type;                     // 0 gated full attention, 1 gated DeltaNet
    int type_index;               // index among the layers of the same type (state / cache / staging slot)
    LinearDesc in_proj;           // [Q|gate|K|V] or [q|k|v|z(|a|b)]
    LinearDesc out_proj;          // row-parallel
    LinearDesc gate_up;           // gate/up interleaved by 8
    LinearDesc down;              // row-parallel
    const void* attn_norm;        // RMSNorm applied to this layer's input
    const void* ffn_norm;         // RMSNorm applied after the attention block
    const void* next_norm;        // RMSNorm applied after the FFN (next layer's input norm / final norm)
    // full attention
    const void* q_norm; const void* k_norm;
    void* kcache; void* vcache;
    // DeltaNet
    const void* wa; const void* wb; const void* conv_w; void* conv_state; float* state;
    const float* A_log; const void* dt_bias; const void* la_norm;
    int off_q, off_k, off_v, off_z, off_a, off_b;
    // FFN on the INT8-activation path (quant_format w8a8 / w4a8): gate, up, down
    int ffn_kind;                 // 0: INT4 weights with fp16 activations, 1: W8A8, 2: W4A8
    int q8_group, q8_F, pad_q8;   // group size of the W4A8 scales; local FFN width
    const void* q8_w[3];          // int8 [N][K] or signed nibbles int32 [N][K/8]
    const void* q8_s[3];          // fp32 [N] (W8A8) or fp16 [K/group][N] (W4A8)
    const void* wab;              // DeltaNet: [wa; wb] as one fp16 [2*nv][H] matrix (many-row steps run it as a GEMM)
};

struct ModelDesc {
    int n_layers, H, vocab, vocab_local, vocab_offset;
    int nq, nkv, hd, rot, rope_interleaved;
    int la_nk, la_nv, la_dk, la_dv;
    int max_seq, max_rows, ar_mode;        // 0 exact, 1 deferred_ref, 2 deferred_consistent
    int attn_splits, argmax_blocks, n_seqs_max;
    float eps;
    int F_pad;                             // padded local FFN width (row stride of the SiLU buffer)
    const void* embed; const void* first_norm;
    LinearDesc lm_head;
    const float* cos_tab; const float* sin_tab;
    // work buffers
    float* h; void* xn; void* proj; int ld_proj; int pad0;
    void* attn_out; int ld_attn; int pad1;
    void* act; float* logits; int ld_logits; int pad2;
    float* gemv_scratch; int* gemv_counters;
    float* attn_scratch; int* attn_counters;
    float* argmax_scratch; int* argmax_counters;
    float* extra; float* h_tmp;            // saved attention partial; uncommitted h + partial (deferred_consistent)
    float* ss; int np; int pad3;           // [rows][np] sums of squares for the lazy RMSNorm
    void* rows; void* rows_tmpl; void* seqs; int* row_tokens; int* seq_rows; int* out_tokens;
    // prefill (many-row) work buffers, sized for max_prefill rows
    int max_prefill; int pad4;
    float* p_h; void* p_xn; void* p_proj; void* p_attn; void* p_act; float* p_partial;
    void* p_rows; void* p_rows_tmpl; int* p_row_tokens; int* tc_status;
    void* p_ab;                            // [max_prefill][2*la_nv] fp16 a/b projections of the DeltaNet layers
    float* coll_gather[B2_MAX_TP]; float* coll_mc_gather; int* coll_counters;
    // many-row steps (batched decode, speculative verification): logits and arg-max scratch for p_logit_rows rows
    float* p_logits; float* p_argmax_scratch; int* p_argmax_counters; int* p_out_tokens;
    float* p_attn_scratch; int* p_attn_counters;     // split-KV scratch for p_logit_rows rows
    int p_logit_rows; int n_lin_layers; int n_full_layers;
    int ab_off;                            // column of p_proj where the a | b gate projections of many-row steps go (-1: none)
    // speculative verification
    SpecStage spec; int* spec_acc; int* spec_result;
    float* state0; void* conv0; long long state_layer_stride, conv_layer_stride;
    void* k0; void* v0; long long kv_layer_stride;
    // sequence-parallel many-row steps (csrc/comm.cu, rs_norm_ag_kernel): p_xn is then this rank's copy of a
    // symmetric buffer, xn_sym its address on every rank, hlast_sym a slot of H floats
    void* xn_sym[B2_MAX_TP]; void* xn_mc; float* hlast_sym[B2_MAX_TP]; int seq_parallel;
    int tagged_splitk;                     // 1: gemv_scratch holds {value, tag} pairs (twice the floats), see GemvInt4Params::tag_word
    // persistent projection chain (csrc/chain.cu)
    void* chain_scratch; unsigned int* chain_counters; int chain_act_cols; int use_chain;
    void* chain_tag_h; void* chain_tag_ss; void* chain_tag_act;
    // INT8-activation FFN work buffers, sized for max(max_rows, max_prefill) rows
    void* q8_xq; float* q8_sx; void* q8_gate; void* q8_up; float* q8_down; void* q8_xn;
    CommCtx comm;
};

// Projections queued for one chain launch, with what the stand-alone GEMV path needs to run them
// instead when the chain kernel cannot take them (fp16 weights, too many rows for shared memory).
struct PendingChain {
    ChainParams cp;
    const LinearDesc* lin[CH_MAX_OPS];
    const LinearDesc* next[CH_MAX_OPS];   // the projection that follows each one in the stream (L2 prefetch hint)
    const void* span[CH_MAX_OPS]; long long span_bytes[CH_MAX_OPS];   // other memory the kernel after it reads first
    int n = 0;
};

struct Driver {
    ModelDesc m;
    std::vector<LayerDesc> layers;
    PendingChain pend;
    long long chain_launches = 0;         // chain kernels issued by the last step that was issued or captured
    long long exchanges = 0;              // cross-GPU exchanges of that step
    std::vector<int> layer_launches;      // kernels issued inside each layer's part of that step
    long long graph_launches = 0, graph_exchanges = 0;   // of the captured step
    long long total_launches = 0, total_exchanges = 0;   // since creation, eager steps and graph replays alike
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int graph_rows = 0, graph_flags = 0;
    long long launches = 0;               // kernels issued by the last eager step
    int scan_prepass = 2;                 // chunked scan: 1 = q / k convolution and norms in a parallel pre-pass,
                                          // 2 = also the state-independent products and the triangle inverse of every chunk
    bool attn_tc = true;                  // prompt attention on tcgen05 (csrc/attention_tc.cu)
    bool gemm_m256 = true;                // 256-output GEMM tiles where the grid stays large enough
    int gemm_m256_min_ctas = 100;
    bool gemm_splitk = true;              // split-K in the many-row GEMMs that add into the residual stream
    const void* pf_span = nullptr; long long pf_span_bytes = 0;   // see run_linear
    bool pf_state = false;                // the in-projection of a DeltaNet layer prefetches that layer's state into L2
    int pf_blocks = 0;                    // k-blocks per warp of the next projection that a GEMV prefetches into L2 (0: off)
    int gemv_seq = 0;                     // split-K GEMVs issued so far in the step being issued (their tags)
    int push_rows_per = 0;                // > 0 while a GEMM is issued whose pushed slices are whole token rows
    bool sp_now = false;                  // the many-row step being issued keeps the residual stream sequence-parallel
};

// The step's generation word: prepare_rows advances it by 1024 at the start of every step, and the n-th
// split-K GEMV of the step tags its partial sums with word + n.  It lives behind the chain kernel's two
// counters in the same small buffer.
static inline unsigned int* step_word(const ModelDesc& m) { return m.chain_counters ? (unsigned int*)m.chain_counters + 4 : nullptr; }

#define STEP_EMBED_TOKENS 1     // gather embeddings from tokens (else: h/xn were loaded by the caller)
#define STEP_LM_HEAD 2          // compute logits
#define STEP_ARGMAX 4           // arg-max into out_tokens (and SeqState.token)
#define STEP_ADVANCE 8          // len += 1 for every row's sequence (plain decode)
#define STEP_NO_COMMIT_DELTA 16 // DeltaNet state dry run
#define STEP_MATERIALIZE_XN 32  // write the final-normed hidden states to xn (hidden-out interface)
#define STEP_SPEC 64            // rows are draft trees: verify without touching the state, accept, commit
#define STEP_GEMM_PATH 128      // many rows: tensor-core GEMMs and the p_* buffers (else the GEMV path, <= 8 rows)

#define CK(x) do { int e_ = (x); if (e_ != 0) return e_; } while (0)

static LazyNorm lazy(const Driver* d, const float* h, const void* w) {
    LazyNorm ln;
    memset(&ln, 0, sizeof(ln));
    ln.h = h; ln.ss = d->m.ss; ln.w = (const __half*)w; ln.np = d->m.np; ln.H = d->m.H; ln.eps = d->m.eps;
    return ln;
}
static LazyNorm no_lazy() { LazyNorm ln; memset(&ln, 0, sizeof(ln)); return ln; }

// next: the INT4 projection that follows in the stream (or null): its first weight blocks are prefetched into
// L2 from inside this launch.  d->pf_span / pf_span_bytes (consumed by the next INT4 launch): a span of memory the
// kernel after this one reads first.
static int run_linear(Driver* d, const LinearDesc& L, const void* x, int ldx, const LazyNorm& ln, int rows,
                      const GemvEpi& epi, cudaStream_t s, const LinearDesc* next = nullptr) {
    d->launches++;
    if (L.kind == LIN_INT4) {
        GemvInt4Params p;
        memset(&p, 0, sizeof(p));
        p.qfrag = (const uint4*)L.w; p.szfrag = (const uint2*)L.sz; p.x = (const __half*)x;
        p.ldx = ldx; p.rows = rows; p.K = L.K; p.KB = L.KB; p.NTL = L.NTL; p.G = L.G;
        p.off32 = L.off32; p.gshift = L.gshift; p.k_splits = L.k_splits; p.L = L.L;
        p.scratch = d->m.gemv_scratch; p.counters = d->m.gemv_counters; p.ln = ln; p.epi = epi; p.comm = d->m.comm;
        if (p.k_splits > 1 && d->gemv_seq < 1023 && d->m.tagged_splitk) { p.tag_word = step_word(d->m); p.tag_base = ++d->gemv_seq; }
        if (d->pf_span) { p.pf_span = d->pf_span; p.pf_span_bytes = d->pf_span_bytes; d->pf_span = nullptr; }
        if (next && next->kind == LIN_INT4 && d->pf_blocks > 0) {
            p.pf_q = (const uint4*)next->w; p.pf_KB = next->KB; p.pf_L = next->L;
            p.pf_nx = next->NTL * 16 / 128; p.pf_ks = next->k_splits; p.pf_blocks = d->pf_blocks;
        }
        return b2_gemv_int4(&p, s);
    }
    GemvF16Params p;
    memset(&p, 0, sizeof(p));
    p.w = (const __half*)L.w; p.x = (const __half*)x; p.ldw = L.ldw; p.ldx = ldx; p.rows = rows;
    p.K = L.K; p.N = L.N; p.k_splits = L.k_splits; p.kslice = L.kslice;
    p.scratch = d->m.gemv_scratch; p.counters = d->m.gemv_counters; p.ln = ln; p.epi = epi; p.comm = d->m.comm;
    return b2_gemv_f16(&p, s);
}

static GemvEpi epi_store(void* out, int ldo, int n_valid, int mode) {
    GemvEpi e;
    memset(&e, 0, sizeof(e));
    e.mode = mode; e.out = out; e.ldo = ldo; e.n_valid = n_valid;
    return e;
}

static GemvEpi epi_finish(Driver* d, int flags, float* hout) {
    GemvEpi e;
    memset(&e, 0, sizeof(e));
    e.mode = EPI_FINISH; e.n_valid = d->m.H; e.fin_flags = flags;
    e.h = d->m.h; e.hout = hout; e.ss_part = d->m.ss; e.extra = d->m.extra; e.eps = d->m.eps;
    e.ss_np = d->m.np;
    return e;
}

// ---- projection chains: consecutive INT4 projections of a step are queued and issued as ONE
// persistent launch (csrc/chain.cu); anything else flushes the queue first.
static int chain_flush(Driver* d, int rows, cudaStream_t s) {
    PendingChain& pc = d->pend;
    if (pc.n == 0) return 0;
    const int n = pc.n;
    pc.n = 0;
    pc.cp.n_ops = n; pc.cp.rows = rows;
    pc.cp.scratch = (float2*)d->m.chain_scratch; pc.cp.counters = d->m.chain_counters;
    pc.cp.tag_h = (float2*)d->m.chain_tag_h; pc.cp.tag_ss = (float2*)d->m.chain_tag_ss; pc.cp.tag_act = (uint2*)d->m.chain_tag_act;
    pc.cp.tag_h_cols = d->m.H; pc.cp.tag_ss_cols = d->m.np; pc.cp.tag_act_cols = d->m.chain_act_cols;
    pc.cp.stages = 0; pc.cp.xf_chunks = 0; pc.cp.pad1 = 0;
    pc.cp.comm = d->m.comm; pc.cp.prof = nullptr;
    if (d->m.use_chain && d->m.chain_scratch && b2_chain_feasible(&pc.cp)) {
        d->launches++; d->chain_launches++;
        return b2_chain(&pc.cp, s);
    }
    for (int i = 0; i < n; ++i) {
        const ChainOp& op = pc.cp.op[i];
        d->pf_span = pc.span[i]; d->pf_span_bytes = pc.span_bytes[i];
        CK(run_linear(d, *pc.lin[i], op.x, op.ldx, op.ln, rows, op.epi, s, pc.next[i]));
        d->pf_span = nullptr;
    }
    return 0;
}

static int chain_add(Driver* d, const LinearDesc& L, const void* x, int ldx, const LazyNorm& ln, int rows,
                     const GemvEpi& epi, cudaStream_t s, const LinearDesc* next = nullptr) {
    const bool exchanges = epi.mode == EPI_FINISH && d->m.comm.tp > 1 && !(epi.fin_flags & FIN_NO_COMM);
    if (exchanges) d->exchanges++;
    // use_chain 2: only the projections that exchange across GPUs go through the chain kernel, each as a
    // launch of its own (its tile-granular exchange is faster than the stand-alone GEMV's finisher); the
    // others stay stand-alone GEMV launches
    if (L.kind != LIN_INT4 || (d->m.use_chain == 2 && !exchanges)) {
        CK(chain_flush(d, rows, s));
        return run_linear(d, L, x, ldx, ln, rows, epi, s, next);
    }
    if (d->m.use_chain == 2) CK(chain_flush(d, rows, s));
    PendingChain& pc = d->pend;
    if (pc.n == CH_MAX_OPS) CK(chain_flush(d, rows, s));
    ChainOp& op = pc.cp.op[pc.n];
    memset(&op, 0, sizeof(op));
    op.qfrag = (const uint4*)L.w; op.szfrag = (const uint2*)L.sz; op.x = (const __half*)x; op.ldx = ldx;
    op.K = L.K; op.KB = L.KB; op.NWT = L.NTL / 4; op.G = L.G; op.off32 = L.off32; op.gshift = L.gshift;
    op.ln = ln; op.epi = epi;
    pc.lin[pc.n] = &L;
    pc.next[pc.n] = next;
    pc.span[pc.n] = d->pf_span; pc.span_bytes[pc.n] = d->pf_span_bytes;
    d->pf_span = nullptr;
    pc.n++;
    if (d->m.use_chain == 2) return chain_flush(d, rows, s);
    return 0;
}

// FFN of one layer on the INT8-activation path (reference: src/inference/engine.py:890-991): the
// normalised input and the SiLU product are quantised per row to int8 in front of the products.
// `h` holds the residual stream the FFN reads and, afterwards, that stream plus the FFN output
// (summed over the ranks); `ss` (optional) receives the row sums of squares for lazy consumers.
static int ffn_q8(Driver* d, const LayerDesc& L, float* h, int rows, float* ss, cudaStream_t s) {
    const ModelDesc& m = d->m;
    if (!m.q8_xq || !L.q8_w[0]) return cudaErrorInvalidValue;
    const int H = m.H, F = L.q8_F;
    CK(b2_add_rmsnorm(h, nullptr, nullptr, L.ffn_norm, m.q8_xn, nullptr, rows, H, m.eps, s)); d->launches++;
    ActQuantParams a;
    memset(&a, 0, sizeof(a));
    a.x = (const __half*)m.q8_xn; a.xq = (int8_t*)m.q8_xq; a.scale = m.q8_sx; a.T = rows; a.K = H; a.ldx = H;
    CK(b2_act_quant(&a, s)); d->launches++;
    auto product = [&](int which, int K, int N, void* out, int f16) -> int {
        Quant8Params q;
        memset(&q, 0, sizeof(q));
        q.w = L.q8_w[which]; q.xq = (const int8_t*)m.q8_xq; q.x_scale = m.q8_sx; q.out = out;
        if (L.ffn_kind == 1) q.w_scale = (const float*)L.q8_s[which]; else q.g_scale = (const __half*)L.q8_s[which];
        q.K = K; q.N = N; q.T = rows; q.ldo = N; q.group = L.q8_group; q.out_f16 = f16; q.w4 = L.ffn_kind == 2;
        d->launches++;
        return b2_linear_q8(&q, s);
    };
    CK(product(0, H, F, m.q8_gate, 1));
    CK(product(1, H, F, m.q8_up, 1));
    CK(b2_silu_mul(m.q8_gate, m.q8_up, m.q8_gate, (size_t)rows * F, s)); d->launches++;
    a.x = (const __half*)m.q8_gate; a.K = F; a.ldx = F;
    CK(b2_act_quant(&a, s)); d->launches++;
    CK(product(2, F, H, m.q8_down, 0));
    if (m.comm.tp > 1) {
        CollParams c;
        memset(&c, 0, sizeof(c));
        c.comm = m.comm; c.in = m.q8_down; c.out = h; c.n = (size_t)rows * H; c.residual = 1;
        c.twoshot = c.n * 4 > 512 * 1024;
        for (int r = 0; r < m.comm.tp; ++r) c.gather[r] = m.coll_gather[r];
        c.mc_gather = m.coll_mc_gather; c.counters = m.coll_counters;
        d->launches++; d->exchanges++;
        CK(b2_allreduce(&c, 2 * 148, s));
        if (ss) { CK(b2_residual_add_ss(h, nullptr, ss, m.np, rows, H, s)); d->launches++; }
    } else if (ss) {
        CK(b2_residual_add_ss(h, m.q8_down, ss, m.np, rows, H, s)); d->launches++;
    } else {
        CK(b2_residual_add(h, m.q8_down, nullptr, (size_t)rows * H, s)); d->launches++;
    }
    return 0;
}

static void fill_delta(const Driver* d, const LayerDesc& L, DeltaParams& q) {
    const ModelDesc& m = d->m;
    memset(&q, 0, sizeof(q));
    q.off_q = L.off_q; q.off_k = L.off_k; q.off_v = L.off_v; q.off_z = L.off_z; q.off_a = L.off_a; q.off_b = L.off_b;
    q.ldx = m.H; q.H = m.H; q.wa = (const __half*)L.wa; q.wb = (const __half*)L.wb;
    q.conv_w = (const __half*)L.conv_w; q.conv_state = (__half*)L.conv_state; q.state = L.state;
    q.A_log = L.A_log; q.dt_bias = (const __half*)L.dt_bias; q.norm_w = (const __half*)L.la_norm;
    q.seq_rows = m.seq_rows; q.ldo = m.ld_attn; q.nk = m.la_nk; q.nv = m.la_nv; q.eps = 1e-6f; q.commit = 1;
}

// After the arg-max of a verify step: accept on the device, then bring DeltaNet states and the
// KV cache to what feeding only the accepted tokens would have left.
static int spec_tail(Driver* d, const void* rows, const int* row_tokens, const int* out_tokens, int n_seqs,
                     cudaStream_t s) {
    const ModelDesc& m = d->m;
    if (!m.spec.base || !m.spec_acc) return cudaErrorInvalidValue;
    SpecAcceptParams a;
    memset(&a, 0, sizeof(a));
    a.out_tokens = out_tokens; a.row_tokens = row_tokens; a.rows = (const RowMeta*)rows; a.seq_rows = m.seq_rows;
    a.seqs = (SeqState*)m.seqs; a.acc = m.spec_acc; a.result = m.spec_result; a.n_seqs = n_seqs;
    CK(b2_spec_accept(&a, s)); d->launches++;
    if (m.n_lin_layers > 0) {
        DeltaCommitParams c;
        memset(&c, 0, sizeof(c));
        c.state0 = m.state0; c.conv0 = (__half*)m.conv0; c.state_layer_stride = m.state_layer_stride;
        c.conv_layer_stride = m.conv_layer_stride; c.st = m.spec; c.acc = m.spec_acc; c.rows = (const RowMeta*)rows;
        c.seq_rows = m.seq_rows; c.nk = m.la_nk; c.nv = m.la_nv; c.n_seqs = n_seqs; c.n_layers = m.n_lin_layers;
        CK(b2_deltanet_commit(&c, m.la_dk, m.la_dv, s)); d->launches++;
    }
    if (m.n_full_layers > 0) {
        KvCompactParams k;
        memset(&k, 0, sizeof(k));
        k.k0 = (__half*)m.k0; k.v0 = (__half*)m.v0; k.layer_stride = m.kv_layer_stride; k.acc = m.spec_acc;
        k.rows = (const RowMeta*)rows; k.seq_rows = m.seq_rows; k.n_layers = m.n_full_layers; k.n_seqs = n_seqs;
        k.nkv = m.nkv; k.hd = m.hd; k.max_seq = m.max_seq;
        CK(b2_kv_compact(&k, s)); d->launches++;
    }
    return 0;
}

static int step_impl(Driver* d, int rows, int n_seqs, int flags, cudaStream_t s) {
    const ModelDesc& m = d->m;
    if (rows < 1 || rows > m.max_rows || rows > B2_MAX_ROWS) return cudaErrorInvalidValue;
    d->launches = 0; d->chain_launches = 0; d->exchanges = 0; d->pend.n = 0;
    const bool tp = m.comm.tp > 1;
    d->gemv_seq = 0;
    CK(b2_prepare_rows(m.rows_tmpl, m.seqs, m.rows, rows, step_word(m), s)); d->launches++;
    if (flags & STEP_EMBED_TOKENS) {
        CK(b2_embed_rmsnorm(m.embed, m.row_tokens, m.rows, m.seqs, m.first_norm, m.h, nullptr, m.ss, m.np, rows,
                            m.H, m.eps, m.vocab, s));
        d->launches++;
    }
    const void* last_norm = m.first_norm;
    for (int li = 0; li < m.n_layers; ++li) {
        const LayerDesc& L = d->layers[li];
        const long long launched0 = d->launches;
        struct Count { Driver* d; int li; long long l0; ~Count() { d->layer_launches[li] = (int)(d->launches - l0); } } count{d, li, launched0};
        const LazyNorm ln_in = lazy(d, m.h, L.attn_norm);
        // ---- token mixer
        // the in-projection rides at the end of the previous layer's chain (out_proj, gate/up, down)
        if (d->pf_state && L.type != 0 && m.n_seqs_max * (long long)m.la_nv * m.la_dk * m.la_dv * 4 <= (8ll << 20)) {
            d->pf_span = L.state; d->pf_span_bytes = m.n_seqs_max * (long long)m.la_nv * m.la_dk * m.la_dv * 4;
        }
        CK(chain_add(d, L.in_proj, nullptr, 0, ln_in, rows, epi_store(m.proj, m.ld_proj, L.in_proj.N, EPI_STORE_F16), s, &L.out_proj));
        d->pf_span = nullptr;
        CK(chain_flush(d, rows, s));
        if (L.type == 0) {
            CK(b2_qknorm_rope_cachew(m.proj, m.ld_proj, m.rows, L.q_norm, L.k_norm, m.cos_tab, m.sin_tab, L.kcache,
                                     L.vcache, rows, m.nq, m.nkv, m.hd, m.rot, m.max_seq, m.rope_interleaved,
                                     m.eps, s));
            d->launches++;
            AttnParams a;
            memset(&a, 0, sizeof(a));
            a.q = (const __half*)m.proj; a.ldq = m.ld_proj; a.gate_off = m.nq * m.hd;
            a.kcache = (const __half*)L.kcache; a.vcache = (const __half*)L.vcache; a.rows = (const RowMeta*)m.rows;
            a.out = (__half*)m.attn_out; a.ldo = m.ld_attn; a.n_rows = rows; a.nq = m.nq; a.nkv = m.nkv;
            a.max_seq = m.max_seq; a.splits = m.attn_splits; a.scale = 1.0f / sqrtf((float)m.hd);
            a.scratch = m.attn_scratch; a.counters = m.attn_counters;
            CK(b2_decode_attn(&a, m.hd, s));
            d->launches++;
        } else {
            DeltaParams q;
            memset(&q, 0, sizeof(q));
            q.proj = (const __half*)m.proj; q.ld = m.ld_proj;
            q.off_q = L.off_q; q.off_k = L.off_k; q.off_v = L.off_v; q.off_z = L.off_z; q.off_a = L.off_a; q.off_b = L.off_b;
            q.xn = nullptr; q.ldx = m.H; q.H = m.H; q.wa = (const __half*)L.wa; q.wb = (const __half*)L.wb;
            q.ln = ln_in;
            q.conv_w = (const __half*)L.conv_w; q.conv_state = (__half*)L.conv_state; q.state = L.state;
            q.A_log = L.A_log; q.dt_bias = (const __half*)L.dt_bias; q.norm_w = (const __half*)L.la_norm;
            q.seq_rows = m.seq_rows; q.rows = (const RowMeta*)m.rows; q.out = (__half*)m.attn_out; q.ldo = m.ld_attn;
            q.nk = m.la_nk; q.nv = m.la_nv; q.n_seqs = n_seqs; q.eps = 1e-6f;
            q.commit = (flags & STEP_NO_COMMIT_DELTA) ? 0 : 1;
            if (flags & STEP_SPEC) CK(b2_deltanet_verify(&q, &m.spec, L.type_index, m.la_dk, m.la_dv, s));
            else CK(b2_deltanet_step(&q, m.la_dk, m.la_dv, s));
            d->launches++;
        }
        int f_attn = 0, f_ffn = 0;
        float* h_mid = m.h;                      // residual stream the FFN reads
        if (!tp) { f_attn = FIN_NO_COMM; f_ffn = FIN_NO_COMM; }
        else if (m.ar_mode == 1) { f_attn = FIN_NO_COMM; }
        else if (m.ar_mode == 2) { f_attn = FIN_NO_COMM | FIN_NO_H_WRITE | FIN_SAVE_EXTRA; f_ffn = FIN_ADD_EXTRA; h_mid = m.h_tmp; }
        CK(chain_add(d, L.out_proj, m.attn_out, m.ld_attn, no_lazy(), rows, epi_finish(d, f_attn, h_mid), s,
                     L.ffn_kind == 0 ? &L.gate_up : nullptr));
        // ---- FFN
        if (L.ffn_kind != 0) {
            if (tp && m.ar_mode != 0) return cudaErrorNotSupported;     // the INT8 path keeps the exact placement
            CK(chain_flush(d, rows, s));
            CK(ffn_q8(d, L, m.h, rows, m.ss, s));
            last_norm = L.next_norm;
            continue;
        }
        CK(chain_add(d, L.gate_up, nullptr, 0, lazy(d, h_mid, L.ffn_norm), rows,
                     epi_store(m.act, m.F_pad, m.F_pad, EPI_SILU_PAIR), s, &L.down));
        CK(chain_add(d, L.down, m.act, m.F_pad, no_lazy(), rows, epi_finish(d, f_ffn, m.h), s,
                     li + 1 < m.n_layers ? &d->layers[li + 1].in_proj : nullptr));
        last_norm = L.next_norm;
    }
    CK(chain_flush(d, rows, s));
    if (flags & STEP_LM_HEAD) {
        CK(run_linear(d, m.lm_head, nullptr, 0, lazy(d, m.h, last_norm), rows,
                      epi_store(m.logits, m.ld_logits, m.vocab_local, EPI_STORE_F32), s));
    }
    if (flags & STEP_MATERIALIZE_XN) {
        CK(b2_add_rmsnorm(m.h, nullptr, nullptr, last_norm, m.xn, nullptr, rows, m.H, m.eps, s));
        d->launches++;
    }
    if (flags & STEP_ARGMAX) {
        ArgmaxParams a;
        memset(&a, 0, sizeof(a));
        a.logits = m.logits; a.ld = m.ld_logits; a.n_rows = rows; a.vocab_local = m.vocab_local;
        a.vocab_offset = m.vocab_offset; a.blocks = m.argmax_blocks; a.scratch = m.argmax_scratch;
        a.counters = m.argmax_counters; a.out_tokens = m.out_tokens;
        a.seqs = (flags & STEP_ADVANCE) ? (SeqState*)m.seqs : nullptr; a.rows = (const RowMeta*)m.rows; a.comm = m.comm;
        CK(b2_argmax(&a, s));
        d->launches++;
    }
    if (flags & STEP_ADVANCE) {
        CK(b2_advance(m.seqs, nullptr, n_seqs, 1, s));
        d->launches++;
    }
    if (flags & STEP_SPEC) {
        // without an arg-max this is a verify-only pass (hidden states out, nothing committed)
        if (flags & STEP_ADVANCE) return cudaErrorInvalidValue;
        if (flags & STEP_ARGMAX) CK(spec_tail(d, m.rows, m.row_tokens, m.out_tokens, n_seqs, s));
    }
    return 0;
}


// ---------------------------------------------------------------------------
// Prefill: T rows of ONE sequence through every layer with tensor-core GEMMs
// (tcgen05), causal attention over the cache, the DeltaNet scan, and -- under
// tensor parallelism -- a two-shot all-reduce fused with the residual add after
// each row-parallel projection.  The reference prefills token-serially through
// its DeltaNet layers and re-launches per-token norm/rope kernels (reference:
// src/inference/tp_engine.py:1900-2224).
// ---------------------------------------------------------------------------
static int run_gemm(Driver* d, const LinearDesc& L, const void* x, int ldx, int T, void* out, int ldo, int n_valid,
                    int epi, cudaStream_t s) {
    if (L.kind != LIN_INT4) return cudaErrorNotSupported;
    GemmTcParams p;
    memset(&p, 0, sizeof(p));
    p.qfrag = (const uint4*)L.w; p.szfrag = (const uint2*)L.sz;
    p.K = L.K; p.KB = L.KB; p.NTL = L.NTL; p.G = L.G; p.off32 = L.off32; p.gshift = L.gshift;
    // tokens per CTA: as many as tensor memory holds, unless that leaves most SMs without a CTA
    // (N = 5120 gives only 40 output tiles): then split the tokens so that the grid fills, but does
    // not exceed, one wave of 148 CTAs (one CTA per SM: a second partial wave would double the time)
    const int ctas_n = L.NTL * 16 / 128;
    int tt = T >= 512 ? 512 : ((T + 15) & ~15);
    int ks = 1;
    if (ctas_n < 148) {
        int parts = 148 / ctas_n;                          // token tiles that still fit one wave
        int need = (T + parts - 1) / parts;
        need = (need + 15) & ~15;
        if (need < 64) need = 64;
        if (need < tt) tt = need;
        if (epi == TC_EPI_RESID_F32 && d->gemm_splitk) {
            // ... or split K instead (the partial products meet in the residual stream through atomic adds):
            // a k-block of a CTA costs about max(0.46, 0.0021 x tokens) us, so few wide token tiles over a
            // third of K beat many narrow ones over all of it.  Pick the cheapest (token tile, splits) pair.
            double best = 1e30;
            const int tmax = T >= 512 ? 512 : ((T + 15) & ~15);
            for (int tiles = 1; tiles <= 8; ++tiles) {
                int t1 = ((T + tiles - 1) / tiles + 15) & ~15;
                if (t1 > tmax) continue;
                if (t1 < 16) t1 = 16;
                const int nt = (T + t1 - 1) / t1;
                int s1 = 148 / (ctas_n * nt);
                if (s1 < 1) continue;
                if (s1 > L.KB / 8) s1 = L.KB / 8 > 0 ? L.KB / 8 : 1;
                const double blk = 0.0021 * t1 > 0.46 ? 0.0021 * t1 : 0.46;
                const double cost = ((L.KB + s1 - 1) / s1) * blk + (s1 > 1 ? 4.0 : 0.0);
                if (cost < best) { best = cost; tt = t1; ks = s1; }
            }
        }
    }
    p.T = T; p.t_tile = tt; p.k_splits = ks;
    // 256-output tiles (two accumulators sharing each activation tile, weights dequantised once for both) where
    // they still give the GPU enough CTAs.
    // Measured (27B, one GPU): with few token rows a weight tile dequantised once for 256 outputs pays (80-row
    // verify step 26.7 -> 26.1 ms); at 512 rows both forms are bound by the shared-memory traffic of the MMA
    // operands and the 256-output form is slightly slower in the prompt (41.9 -> 42.5 ms), so it is used below
    // 256 rows only.
    if (d->gemm_m256 && T < 256 && (L.NTL * 16) % 256 == 0 &&
        (epi == TC_EPI_STORE_F16 || epi == TC_EPI_SILU_PAIR || epi == TC_EPI_STORE_F32)) {
        const int tt2 = T >= 256 ? 256 : ((T + 15) & ~15);
        const int ctas = (L.NTL * 16 / 256) * ((T + tt2 - 1) / tt2);
        if (ctas >= d->gemm_m256_min_ctas) { p.m_halves = 2; p.t_tile = tt2; p.k_splits = 1; }
    }
    p.n_valid = n_valid; p.ldo = ldo; p.epi = epi; p.out = out; p.status = d->m.tc_status;
    if (epi == TC_EPI_PUSH_F32) {
        const CommCtx& c = d->m.comm;
        const size_t n4 = (size_t)T * ldo / 4;
        for (int r = 0; r < c.tp; ++r) p.push[r] = c.part[r];
        p.epoch = c.epoch; p.part_stride = (long long)c.part_stride;
        p.push_tp = c.tp; p.push_rank = c.rank; p.push_per = (unsigned)((n4 + c.tp - 1) / c.tp);
        if (d->push_rows_per > 0) p.push_per = (unsigned)((size_t)d->push_rows_per * ldo / 4);    // slices of whole token rows
    }
    d->launches++;
    return b2_gemm_int4_tc(&p, x, ldx, s);
}

// True when the many-row step keeps the residual stream sequence-parallel: each row-parallel projection is
// followed by one kernel that reduce-scatters by token rows, adds the residual, applies the NEXT RMSNorm and
// all-gathers the fp16 result (so the callers skip their add_rmsnorm launches).
static bool seq_parallel_rows(const ModelDesc& m, int T) {
    if (m.comm.tp <= 1 || !m.seq_parallel) return false;
    const int per = (T + m.comm.tp - 1) / m.comm.tp;
    return (size_t)m.comm.tp * per * m.H <= (size_t)m.comm.part_stride && m.H % 8 == 0 && m.H <= 8192;
}

static int row_parallel(Driver* d, const LinearDesc& L, const void* x, int ldx, int T, const void* next_norm, cudaStream_t s) {
    const ModelDesc& m = d->m;
    if (m.comm.tp <= 1) return run_gemm(d, L, x, ldx, T, m.p_h, m.H, m.H, TC_EPI_RESID_F32, s);
    if (d->sp_now) {
        const int per = (T + m.comm.tp - 1) / m.comm.tp;
        d->push_rows_per = per;
        CK(run_gemm(d, L, x, ldx, T, nullptr, m.H, m.H, TC_EPI_PUSH_F32, s));
        d->push_rows_per = 0;
        SeqParParams q;
        memset(&q, 0, sizeof(q));
        q.comm = m.comm; q.h = m.p_h; q.norm_w = (const __half*)next_norm;
        for (int r = 0; r < m.comm.tp; ++r) { q.xn[r] = (__half*)m.xn_sym[r]; q.hlast[r] = m.hlast_sym[r]; }
        q.mc_xn = (__half*)m.xn_mc;
        q.T = T; q.H = m.H; q.rows_per = per; q.eps = m.eps; q.counters = m.coll_counters;
        d->launches++; d->exchanges++;
        return b2_rs_norm_ag(&q, s);
    }
    // Tensor parallel: the GEMM epilogue pushes every output tile into the staging buffer of the rank
    // that reduces that slice (reduce-scatter traffic overlaps the GEMM); the collective kernel then
    // sums its slice from local memory, multicasts it, and adds the residual.
    CK(run_gemm(d, L, x, ldx, T, nullptr, m.H, m.H, TC_EPI_PUSH_F32, s));
    CollParams c;
    memset(&c, 0, sizeof(c));
    c.comm = m.comm; c.in = nullptr; c.out = m.p_h; c.n = (size_t)T * m.H; c.residual = 1;
    c.twoshot = 1; c.pushed = 1;
    for (int r = 0; r < m.comm.tp; ++r) c.gather[r] = m.coll_gather[r];
    c.mc_gather = m.coll_mc_gather; c.counters = m.coll_counters;
    d->launches++; d->exchanges++;
    return b2_allreduce(&c, 2 * 148, s);
}

static int rows_impl(Driver* d, int T, int n_seqs, int flags, cudaStream_t s) {
    const ModelDesc& m = d->m;
    if (T < 1 || T > m.max_prefill) return cudaErrorInvalidValue;
    d->launches = 0; d->chain_launches = 0; d->exchanges = 0;
    d->gemv_seq = 0;
    CK(b2_prepare_rows(m.p_rows_tmpl, m.seqs, m.p_rows, T, step_word(m), s)); d->launches++;
    if (flags & STEP_EMBED_TOKENS) {
        CK(b2_embed_rmsnorm(m.embed, m.p_row_tokens, m.p_rows, m.seqs, m.first_norm, m.p_h, m.p_xn, nullptr, 0, T,
                            m.H, m.eps, m.vocab, s));
        d->launches++;
    }
    // sequence-parallel residual stream: not with INT8-activation FFNs (their kernels read full residual rows)
    bool sp = seq_parallel_rows(m, T);
    for (int li = 0; li < m.n_layers && sp; ++li) if (d->layers[li].ffn_kind != 0) sp = false;
    d->sp_now = sp;
    for (int li = 0; li < m.n_layers; ++li) {
        const LayerDesc& L = d->layers[li];
        struct Count { Driver* d; int li; long long l0; ~Count() { d->layer_launches[li] = (int)(d->launches - l0); } } count{d, li, d->launches};
        if (li > 0 && !sp) { CK(b2_add_rmsnorm(m.p_h, nullptr, nullptr, L.attn_norm, m.p_xn, nullptr, T, m.H, m.eps, s)); d->launches++; }
        CK(run_gemm(d, L.in_proj, m.p_xn, m.H, T, m.p_proj, m.ld_proj, L.in_proj.N, TC_EPI_STORE_F16, s));
        if (L.type == 0) {
            CK(b2_qknorm_rope_cachew(m.p_proj, m.ld_proj, m.p_rows, L.q_norm, L.k_norm, m.cos_tab, m.sin_tab, L.kcache,
                                     L.vcache, T, m.nq, m.nkv, m.hd, m.rot, m.max_seq, m.rope_interleaved, m.eps, s));
            AttnParams a;
            memset(&a, 0, sizeof(a));
            a.q = (const __half*)m.p_proj; a.ldq = m.ld_proj; a.gate_off = m.nq * m.hd;
            a.kcache = (const __half*)L.kcache; a.vcache = (const __half*)L.vcache; a.rows = (const RowMeta*)m.p_rows;
            a.out = (__half*)m.p_attn; a.ldo = m.ld_attn; a.n_rows = T; a.nq = m.nq; a.nkv = m.nkv;
            a.max_seq = m.max_seq; a.scale = 1.0f / sqrtf((float)m.hd);
            // tensor-core attention over 16-row tiles; few tiles with long contexts (batched decode,
            // verification) are cut into cache slices so that the GPU fills, a prompt's many tiles are not
            a.splits = 1; a.scratch = m.attn_scratch; a.counters = m.attn_counters;
            if (T <= m.p_logit_rows && m.p_attn_scratch) {
                const int tiles = (T + 15) / 16 > n_seqs ? (T + 15) / 16 : n_seqs;
                int sp = 148 / (tiles * m.nkv);
                sp = sp < 1 ? 1 : (sp > m.attn_splits ? m.attn_splits : sp);
                a.splits = sp; a.scratch = m.p_attn_scratch;
            }
            if (!(flags & STEP_SPEC) && n_seqs == 1 && T >= 64 && d->attn_tc) {
                // a prompt chunk of one sequence: QK^T and PV on tcgen05 with TMA-fed Q / K tiles
                a.splits = 1;
                CK(b2_attn_prefill_tc(&a, 0, T, m.n_seqs_max, m.hd, m.tc_status, s));
                d->launches += 2;
            } else {
                CK(b2_attn_rows(&a, m.seq_rows, n_seqs, m.hd, s));
                d->launches += a.splits > 1 ? 3 : 2;
            }
        } else {
            DeltaParams q;
            fill_delta(d, L, q);
            q.proj = (const __half*)m.p_proj; q.ld = m.ld_proj; q.xn = (const __half*)m.p_xn;
            q.rows = (const RowMeta*)m.p_rows; q.out = (__half*)m.p_attn; q.n_seqs = n_seqs;
            // the tiny a/b gate projections: from the in-projection if the checkpoint quantised them with it,
            // else one small dense kernel for all rows into spare columns of the projection buffer
            const void* ab = (const __half*)m.p_proj + (L.off_a >= 0 ? L.off_a : 0);
            if (L.off_a < 0 && m.ab_off >= 0) {
                if (L.wab && T >= 64 && m.H % 64 == 0) {
                    // the two small gate projections of all rows as one dense tensor-core GEMM (weights by TMA)
                    GemmTcParams g;
                    memset(&g, 0, sizeof(g));
                    g.K = m.H; g.T = T; g.t_tile = 64;
                    g.n_valid = 2 * m.la_nv; g.ldo = m.ld_proj; g.epi = TC_EPI_STORE_F16;
                    g.out = (__half*)m.p_proj + m.ab_off; g.status = m.tc_status;
                    CK(b2_gemm_f16_tc(&g, L.wab, m.H, m.p_xn, m.H, s));
                } else {
                    CK(b2_ab_proj(m.p_xn, m.H, L.wa, L.wb, m.la_nv, m.H, (__half*)m.p_proj + m.ab_off, m.ld_proj, T, s));
                }
                d->launches++;
                ab = (const __half*)m.p_proj + m.ab_off;
                q.off_a = m.ab_off; q.off_b = m.ab_off + m.la_nv;
            }
            if (flags & STEP_SPEC) {
                CK(b2_deltanet_verify(&q, &m.spec, L.type_index, m.la_dk, m.la_dv, s));
            } else if (n_seqs == 1 && T >= 16) {
                // the FFN activation buffer is idle here: it holds the outputs of the two pre-passes (q | k of all rows,
                // then T | W of every chunk and value head) when it is large enough
                const int ld_qk = 2 * m.la_nk * m.la_dk;
                const size_t cap = (size_t)m.max_prefill * m.F_pad * sizeof(__half);
                const size_t qk_bytes = (((size_t)T * ld_qk * sizeof(__half)) + 255) & ~(size_t)255;
                const size_t tw_bytes = (size_t)b2_deltanet_tw_floats(m.la_nv, T) * sizeof(float);
                void* qk = (d->scan_prepass && qk_bytes <= cap) ? m.p_act : nullptr;
                void* tw = (qk && d->scan_prepass > 1 && qk_bytes + tw_bytes <= cap) ? (void*)((char*)m.p_act + qk_bytes) : nullptr;
                CK(b2_deltanet_chunk(&q, ab, m.ld_proj, qk, ld_qk, T, tw, m.la_dk, m.la_dv, s));
                if (qk) d->launches++;
                if (tw) d->launches++;
            } else {
                CK(b2_deltanet_step(&q, m.la_dk, m.la_dv, s));
            }
            d->launches++;
        }
        // prefill always uses the exact all-reduce placement
        CK(row_parallel(d, L.out_proj, m.p_attn, m.ld_attn, T, L.ffn_norm, s));
        if (L.ffn_kind != 0) { CK(ffn_q8(d, L, m.p_h, T, nullptr, s)); continue; }
        if (!sp) { CK(b2_add_rmsnorm(m.p_h, nullptr, nullptr, L.ffn_norm, m.p_xn, nullptr, T, m.H, m.eps, s)); d->launches++; }
        CK(run_gemm(d, L.gate_up, m.p_xn, m.H, T, m.p_act, m.F_pad, m.F_pad, TC_EPI_SILU_PAIR, s));
        CK(row_parallel(d, L.down, m.p_act, m.F_pad, T, L.next_norm, s));
    }
    // final norm of every row (hidden-out interface and the lm_head input)
    if (!sp) {
        CK(b2_add_rmsnorm(m.p_h, nullptr, nullptr, d->layers[m.n_layers - 1].next_norm, m.p_xn, nullptr, T, m.H, m.eps, s));
        d->launches++;
    }
    if (flags & STEP_LM_HEAD) {
        // logits of every row: the fp16 lm_head goes through the same tcgen05 pipeline, weights by TMA
        if (T > m.p_logit_rows || m.lm_head.kind != LIN_F16) return cudaErrorInvalidValue;
        GemmTcParams g;
        memset(&g, 0, sizeof(g));
        g.K = m.lm_head.K; g.T = T; g.t_tile = T >= 512 ? 512 : ((T + 15) & ~15);
        g.n_valid = m.vocab_local; g.ldo = m.ld_logits; g.epi = TC_EPI_STORE_F32; g.out = m.p_logits; g.status = m.tc_status;
        CK(b2_gemm_f16_tc(&g, m.lm_head.w, m.lm_head.ldw, m.p_xn, m.H, s));
        d->launches++;
    }
    if (flags & STEP_ARGMAX) {
        if (!(flags & STEP_LM_HEAD)) return cudaErrorInvalidValue;
        ArgmaxParams a;
        memset(&a, 0, sizeof(a));
        a.logits = m.p_logits; a.ld = m.ld_logits; a.n_rows = T; a.vocab_local = m.vocab_local;
        a.vocab_offset = m.vocab_offset; a.blocks = m.argmax_blocks; a.scratch = m.p_argmax_scratch;
        a.counters = m.p_argmax_counters; a.out_tokens = m.p_out_tokens;
        a.seqs = (flags & STEP_ADVANCE) ? (SeqState*)m.seqs : nullptr; a.rows = (const RowMeta*)m.p_rows; a.comm = m.comm;
        CK(b2_argmax(&a, s));
        d->launches++;
    }
    if (flags & STEP_ADVANCE) {
        CK(b2_advance(m.seqs, nullptr, n_seqs, 1, s));
        d->launches++;
    }
    if (flags & STEP_SPEC) {
        if (flags & STEP_ADVANCE) return cudaErrorInvalidValue;
        if (flags & STEP_ARGMAX) CK(spec_tail(d, m.p_rows, m.p_row_tokens, m.p_out_tokens, n_seqs, s));
    }
    return 0;
}

static int run_impl(Driver* d, int rows, int n_seqs, int flags, cudaStream_t s) {
    return (flags & STEP_GEMM_PATH) ? rows_impl(d, rows, n_seqs, flags, s) : step_impl(d, rows, n_seqs, flags, s);
}

static int counted(Driver* d, int rc) {
    d->total_launches += d->launches; d->total_exchanges += d->exchanges;
    return rc;
}
B2_API int b2_driver_prefill(void* h, int T, int flags, cudaStream_t s) { return counted((Driver*)h, rows_impl((Driver*)h, T, 1, flags, s)); }
B2_API int b2_driver_rows(void* h, int T, int n_seqs, int flags, cudaStream_t s) {
    return counted((Driver*)h, rows_impl((Driver*)h, T, n_seqs, flags, s));
}

B2_API void* b2_driver_create(const ModelDesc* m, const LayerDesc* layers) {
    Driver* d = new Driver();
    d->m = *m;
    d->layers.assign(layers, layers + m->n_layers);
    d->layer_launches.assign(m->n_layers, 0);
    // Off by default: measured on B200 (27B, one GPU, tg128) 213.6 tok/s with 4 blocks per warp, 213.1 with 2,
    // 208.7 with 8, against 213.9 without: the gaps between GEMVs are not waiting on HBM.
    const char* g256 = getenv("B200GRAD_GEMM_M256");
    d->gemm_m256 = !(g256 && atoi(g256) == 0);
    if (g256 && atoi(g256) > 1) d->gemm_m256_min_ctas = atoi(g256);
    const char* gsk = getenv("B200GRAD_GEMM_SPLITK");
    d->gemm_splitk = !(gsk && atoi(gsk) == 0);
    const char* spp = getenv("B200GRAD_SCAN_PREPASS");
    d->scan_prepass = spp ? atoi(spp) : 2;
    const char* atc = getenv("B200GRAD_ATTN_TC");
    d->attn_tc = !(atc && atoi(atc) == 0);
    // Off by default: 214.73 against 214.30 tok/s (27B, one GPU, two runs each): the DeltaNet step's wait for its
    // state is a small part of its 10 us.
    const char* pfs = getenv("B200GRAD_PREFETCH_STATE");
    d->pf_state = pfs && atoi(pfs) != 0;
    const char* pf = getenv("B200GRAD_L2_PREFETCH");
    d->pf_blocks = pf ? atoi(pf) : 0;
    return d;
}
B2_API void b2_driver_destroy(void* h) {
    Driver* d = (Driver*)h;
    if (!d) return;
    if (d->exec) cudaGraphExecDestroy(d->exec);
    if (d->graph) cudaGraphDestroy(d->graph);
    delete d;
}
B2_API int b2_driver_step(void* h, int rows, int n_seqs, int flags, cudaStream_t s) {
    return counted((Driver*)h, run_impl((Driver*)h, rows, n_seqs, flags, s));
}
B2_API long long b2_driver_total_launches(void* h) { return ((Driver*)h)->total_launches; }
B2_API long long b2_driver_total_exchanges(void* h) { return ((Driver*)h)->total_exchanges; }
B2_API long long b2_driver_launches(void* h) { return ((Driver*)h)->launches; }
B2_API long long b2_driver_chain_launches(void* h) { return ((Driver*)h)->chain_launches; }
B2_API long long b2_driver_exchanges(void* h) { return ((Driver*)h)->exchanges; }
B2_API int b2_driver_layer_launches(void* h, int layer) {
    Driver* d = (Driver*)h;
    return layer >= 0 && layer < (int)d->layer_launches.size() ? d->layer_launches[layer] : -1;
}

// Capture one step into a graph (the stream must be a non-default stream).
B2_API int b2_driver_capture(void* h, int rows, int n_seqs, int flags, cudaStream_t s) {
    Driver* d = (Driver*)h;
    if (d->exec) { cudaGraphExecDestroy(d->exec); d->exec = nullptr; }
    if (d->graph) { cudaGraphDestroy(d->graph); d->graph = nullptr; }
    cudaError_t e = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) return e;
    int r = run_impl(d, rows, n_seqs, flags, s);
    cudaGraph_t g = nullptr;
    e = cudaStreamEndCapture(s, &g);
    if (r != 0) { if (g) cudaGraphDestroy(g); return r; }
    if (e != cudaSuccess) return e;
    d->graph = g;
    e = cudaGraphInstantiate(&d->exec, g, 0);
    if (e != cudaSuccess) return e;
    d->graph_rows = rows; d->graph_flags = flags;
    d->graph_launches = d->launches; d->graph_exchanges = d->exchanges;
    return 0;
}
// Replay the captured step `n` times back to back.
B2_API int b2_driver_replay(void* h, int n, cudaStream_t s) {
    Driver* d = (Driver*)h;
    if (!d->exec) return cudaErrorInvalidValue;
    for (int i = 0; i < n; ++i) {
        cudaError_t e = cudaGraphLaunch(d->exec, s);
        if (e != cudaSuccess) return e;
        d->total_launches += d->graph_launches; d->total_exchanges += d->graph_exchanges;
    }
    return 0;
}
B2_API int b2_driver_graph_nodes(void* h) {
    Driver* d = (Driver*)h;
    size_t n = 0;
    if (!d->graph || cudaGraphGetNodes(d->graph, nullptr, &n) != cudaSuccess) return -1;
    return (int)n;
}
B2_API int b2_sizeof_linear_desc() { return (int)sizeof(LinearDesc); }
B2_API int b2_sizeof_layer_desc() { return (int)sizeof(LayerDesc); }
B2_API int b2_sizeof_model_desc() { return (int)sizeof(ModelDesc); }
B2_API int b2_sizeof_row_meta() { return (int)sizeof(RowMeta); }
B2_API int b2_sizeof_seq_state() { return (int)sizeof(SeqState); }
