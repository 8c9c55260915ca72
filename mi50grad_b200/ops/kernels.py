"""Python entry points of the individual CUDA kernels (used by the tests, the
micro-benchmarks and the parts of the engines that run outside the step driver).
Every function launches on the current CUDA stream and raises if the launch
fails; there is no PyTorch fallback."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import lib as L


def _vp(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def make_rows(entries, device) -> torch.Tensor:
    """entries: (seq, pos, slot, ctx, mask) per row -> device RowMeta array."""
    t = torch.zeros(len(entries), 6, dtype=torch.int32)
    for r, (seq, pos, slot, ctx, mask) in enumerate(entries):
        t[r, 0], t[r, 1], t[r, 2], t[r, 3] = seq, pos, slot, ctx
        lo, hi = mask & 0xFFFFFFFF, (mask >> 32) & 0xFFFFFFFF
        t[r, 4] = lo - (1 << 32 if lo & 0x80000000 else 0)
        t[r, 5] = hi - (1 << 32 if hi & 0x80000000 else 0)
    return t.to(device)


def _epi(mode, out=None, ldo=0, n_valid=0, fin_flags=0, h=None, norm_w=None, xn=None, extra=None,
         hout=None, ss_part=None, eps=1e-6) -> L.GemvEpi:
    e = L.GemvEpi()
    e.mode, e.ldo, e.n_valid, e.fin_flags = mode, ldo, n_valid, fin_flags
    e.out, e.h, e.norm_w, e.xn = L.ptr(out), L.ptr(h), L.ptr(norm_w), L.ptr(xn)
    e.extra, e.eps = L.ptr(extra), eps
    e.hout = L.ptr(hout if hout is not None else h)
    e.ss_part = L.ptr(ss_part)
    return e


def lazy_norm(h: torch.Tensor, ss: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> L.LazyNorm:
    """Input descriptor: x = h * rsqrt(sum(ss[row]) / H + eps) * w, formed by the consumer."""
    ln = L.LazyNorm()
    ln.h, ln.ss, ln.w = h.data_ptr(), ss.data_ptr(), w.data_ptr()
    ln.np, ln.H, ln.eps = ss.shape[1], h.shape[1], eps
    return ln


def gemv(lin, x: Optional[torch.Tensor], out: Optional[torch.Tensor] = None, mode: int = L.EPI_STORE_F16,
         scratch: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None,
         comm: Optional[L.CommCtx] = None, fin_flags: int = 0, h=None, norm_w=None, xn=None,
         extra=None, hout=None, ss_part=None, eps: float = 1e-6, n_valid: Optional[int] = None,
         k_splits: Optional[int] = None, Lblocks: Optional[int] = None, ln: Optional[L.LazyNorm] = None,
         rows: Optional[int] = None):
    """y = x W^T for x[rows, K] fp16 (or a lazily normalised fp32 stream `ln`) with a
    `DeviceLinear`-like object (`.packed` PackedInt4 or `.dense` fp16 [N, K]) and one of
    the four epilogues.  EPI_FINISH: hout = h + y (+ all-reduce), ss_part = per-tile
    sums of squares of hout (one total and zeros after an exchange)."""
    lib = L.lib()
    rows = x.shape[0] if x is not None else rows
    dev = x.device if x is not None else (out if out is not None else h).device
    pk, dense = getattr(lin, "packed", None), getattr(lin, "dense", None)
    if pk is None and dense is None:
        pk = lin
    ks = k_splits or (pk.k_splits if pk is not None else lin.k_splits)
    n_pad = pk.n_pad if pk is not None else -(-dense.shape[0] // 128) * 128
    if scratch is None:
        scratch = torch.empty(max(1, ks * rows * n_pad), dtype=torch.float32, device=dev)
    if counters is None:
        counters = torch.zeros(n_pad // 128 + 2, dtype=torch.int32, device=dev)
    N = pk.N if pk is not None else dense.shape[0]
    if mode == L.EPI_SILU_PAIR:
        nv = n_valid if n_valid is not None else n_pad // 2
    elif mode == L.EPI_FINISH:
        nv = N
    else:
        nv = n_valid if n_valid is not None else N
    if mode == L.EPI_FINISH and ss_part is None:
        ss_part = torch.zeros(rows, -(-N // 128), dtype=torch.float32, device=dev)
    epi = _epi(mode, out, out.stride(0) if out is not None else 0, nv, fin_flags, h, norm_w, xn, extra,
               hout, ss_part, eps)
    xptr = x.data_ptr() if x is not None else None
    ldx = x.stride(0) if x is not None else 0
    cm = comm if comm is not None else L.null_comm()
    if pk is not None:
        p = L.GemvInt4Params()
        p.qfrag, p.szfrag, p.x = pk.qfrag.data_ptr(), pk.szfrag.data_ptr(), xptr
        p.ldx, p.rows, p.K, p.KB, p.NTL, p.G = ldx, rows, pk.K, pk.KB, pk.NTL, pk.G
        if ln is not None:
            p.ln = ln
        p.off32, p.gshift, p.k_splits, p.L = pk.off32, pk.gshift, ks, Lblocks or pk.L
        if k_splits and not Lblocks:
            p.L = -(-pk.KB // (4 * ks))
        p.scratch, p.counters, p.epi, p.comm = scratch.data_ptr(), counters.data_ptr(), epi, cm
        L.check(lib.b2_gemv_int4(C.byref(p), L.stream()), "gemv_int4")
    else:
        p = L.GemvF16Params()
        p.w, p.x, p.ldw, p.ldx, p.rows = dense.data_ptr(), xptr, dense.stride(0), ldx, rows
        if ln is not None:
            p.ln = ln
        p.K, p.N, p.k_splits, p.kslice = dense.shape[1], dense.shape[0], ks, lin.kslice
        p.scratch, p.counters, p.epi, p.comm = scratch.data_ptr(), counters.data_ptr(), epi, cm
        L.check(lib.b2_gemv_f16(C.byref(p), L.stream()), "gemv_f16")
    return ss_part if mode == L.EPI_FINISH else out


def chain_op(pk, x: Optional[torch.Tensor] = None, ln: Optional[L.LazyNorm] = None, mode: int = L.EPI_STORE_F16,
             out: Optional[torch.Tensor] = None, n_valid: Optional[int] = None, fin_flags: int = 0, h=None,
             hout=None, extra=None, ss_part=None, eps: float = 1e-6) -> L.ChainOp:
    """One projection of a `chain` launch: `pk` is a PackedInt4, the input either fp16 rows `x` or a
    lazily normalised stream `ln`, the epilogue as in `gemv` (FINISH tiles are 64 columns wide:
    `ss_part` is [rows, >= N/64])."""
    op = L.ChainOp()
    op.qfrag, op.szfrag = pk.qfrag.data_ptr(), pk.szfrag.data_ptr()
    op.x, op.ldx = (x.data_ptr(), x.stride(0)) if x is not None else (None, 0)
    op.K, op.KB, op.NWT, op.G, op.off32, op.gshift = pk.K, pk.KB, pk.NTL // 4, pk.G, pk.off32, pk.gshift
    if ln is not None:
        op.ln = ln
    if mode == L.EPI_SILU_PAIR:
        nv = n_valid if n_valid is not None else pk.n_pad // 2
    elif mode == L.EPI_FINISH:
        nv = pk.N
    else:
        nv = n_valid if n_valid is not None else pk.N
    op.epi = _epi(mode, out, out.stride(0) if out is not None else 0, nv, fin_flags, h, None, None, extra,
                  hout, ss_part, eps)
    if ss_part is not None:
        op.epi.ss_np = ss_part.shape[1]
    return op


class ChainBuffers:
    """Work buffers of `chain` launches over a set of projections: cross-CTA scratch, the launch
    counters, and the tagged hand-off buffers between the projections of one launch."""

    def __init__(self, ops, rows: int, device):
        lib = L.lib()
        need = max(int(lib.b2_chain_scratch_floats(o.KB, o.NWT, rows)) for o in ops)
        self.rows = rows
        self.scratch = torch.zeros(max(2, need), dtype=torch.float32, device=device)
        self.counters = torch.zeros(8, dtype=torch.int32, device=device)
        self.h_cols = max([o.epi.n_valid for o in ops if o.epi.mode == L.EPI_FINISH] + [2])
        self.h_cols += self.h_cols & 1
        self.ss_cols = max([o.NWT for o in ops if o.epi.mode == L.EPI_FINISH] + [1])
        self.act_cols = max([-(-o.epi.n_valid // 2) for o in ops if o.epi.mode == L.EPI_SILU_PAIR] + [1])
        self.tag_h = torch.zeros(rows, self.h_cols, 2, dtype=torch.float32, device=device)
        self.tag_ss = torch.zeros(rows, self.ss_cols, 2, dtype=torch.float32, device=device)
        self.tag_act = torch.zeros(rows, self.act_cols, 2, dtype=torch.int32, device=device)


def chain_scratch(ops, rows: int, device) -> ChainBuffers:
    return ChainBuffers(ops, rows, device)


def chain(ops, rows: int, bufs: ChainBuffers, comm: Optional[L.CommCtx] = None, prof: Optional[torch.Tensor] = None):
    """Run up to four dependent INT4 projections (`chain_op`) as ONE persistent launch
    (csrc/chain.cu): each projection must read what its predecessor writes.  Raises if they
    cannot run as one launch (shapes, or rows x K too large for shared memory)."""
    lib = L.lib()
    p = L.ChainParams()
    p.n_ops, p.rows = len(ops), rows
    for i, o in enumerate(ops):
        p.op[i] = o
    p.scratch, p.counters = bufs.scratch.data_ptr(), bufs.counters.data_ptr()
    p.tag_h, p.tag_ss, p.tag_act = bufs.tag_h.data_ptr(), bufs.tag_ss.data_ptr(), bufs.tag_act.data_ptr()
    p.tag_h_cols, p.tag_ss_cols, p.tag_act_cols = bufs.h_cols, bufs.ss_cols, bufs.act_cols
    p.prof = None if prof is None else prof.data_ptr()     # int64 [SMs * 8 warps, 4, 8] per-warp timing record
    p.comm = comm if comm is not None else L.null_comm()
    if not lib.b2_chain_feasible(C.byref(p)):
        raise ValueError("projection chain does not fit one launch (rows x K too large for shared memory, or "
                         "projections that do not feed one another)")
    L.check(lib.b2_chain(C.byref(p), L.stream()), "chain")


def add_rmsnorm(h: torch.Tensor, w: torch.Tensor, delta: Optional[torch.Tensor] = None, eps: float = 1e-6,
                out32: bool = False):
    """h (fp32 [rows, H]) += delta; returns rmsnorm(h)*w as fp16 (or fp32)."""
    rows, H = h.shape
    xn = torch.empty(rows, H, dtype=torch.float32 if out32 else torch.float16, device=h.device)
    d32 = delta if delta is not None and delta.dtype == torch.float32 else None
    d16 = delta if delta is not None and delta.dtype == torch.float16 else None
    L.check(L.lib().b2_add_rmsnorm(_vp(h), _vp(d32), _vp(d16), _vp(w), None if out32 else _vp(xn),
                                   _vp(xn) if out32 else None, rows, H, C.c_float(eps), L.stream()), "add_rmsnorm")
    return xn


def embed_rmsnorm(embed, row_tokens, rows_meta, seqs, w, h, xn=None, ss_part=None, eps=1e-6):
    n, H = h.shape
    np_ = ss_part.shape[1] if ss_part is not None else 0
    L.check(L.lib().b2_embed_rmsnorm(_vp(embed), _vp(row_tokens), _vp(rows_meta), _vp(seqs), _vp(w), _vp(h),
                                     _vp(xn), _vp(ss_part), np_, n, H, C.c_float(eps), embed.shape[0],
                                     L.stream()), "embed_rmsnorm")


def qknorm_rope_cachew(qkv, rows_meta, q_norm, k_norm, cos_tab, sin_tab, kcache, vcache, nq, nkv, hd, rot,
                       interleaved=True, eps=1e-6):
    """kcache/vcache: [seqs, max_seq, nkv, hd] fp16."""
    L.check(L.lib().b2_qknorm_rope_cachew(_vp(qkv), qkv.stride(0), _vp(rows_meta), _vp(q_norm), _vp(k_norm),
                                          _vp(cos_tab), _vp(sin_tab), _vp(kcache), _vp(vcache), qkv.shape[0], nq,
                                          nkv, hd, rot, kcache.shape[1], 1 if interleaved else 0, C.c_float(eps),
                                          L.stream()), "qknorm_rope_cachew")


def decode_attn(q, rows_meta, kcache, vcache, nq, nkv, hd, gate_off=-1, splits=4, out=None):
    n = q.shape[0]
    dev = q.device
    if out is None:
        out = torch.empty(n, nq * hd, dtype=torch.float16, device=dev)
    G = nq // nkv
    p = L.AttnParams()
    p.q, p.ldq, p.gate_off = q.data_ptr(), q.stride(0), gate_off
    p.kcache, p.vcache, p.rows = kcache.data_ptr(), vcache.data_ptr(), rows_meta.data_ptr()
    p.out, p.ldo, p.n_rows, p.nq, p.nkv = out.data_ptr(), out.stride(0), n, nq, nkv
    p.max_seq, p.splits, p.scale = kcache.shape[1], splits, 1.0 / hd ** 0.5
    scratch = torch.empty(n * nkv * splits * G * (hd + 4), dtype=torch.float32, device=dev)
    counters = torch.zeros(n * nkv + 1, dtype=torch.int32, device=dev)
    p.scratch, p.counters = scratch.data_ptr(), counters.data_ptr()
    L.check(L.lib().b2_decode_attn(C.byref(p), hd, L.stream()), "decode_attn")
    return out


def attn_rows(q, rows_meta, seq_rows, kcache, vcache, nq, nkv, hd, gate_off=-1, splits=1, out=None):
    """Tensor-core attention for many rows (16-row tiles per sequence); seq_rows: int32 [n_seqs+1]."""
    n = q.shape[0]
    dev = q.device
    if out is None:
        out = torch.empty(n, nq * hd, dtype=torch.float16, device=dev)
    p = L.AttnParams()
    p.q, p.ldq, p.gate_off = q.data_ptr(), q.stride(0), gate_off
    p.kcache, p.vcache, p.rows = kcache.data_ptr(), vcache.data_ptr(), rows_meta.data_ptr()
    p.out, p.ldo, p.n_rows, p.nq, p.nkv = out.data_ptr(), out.stride(0), n, nq, nkv
    p.max_seq, p.splits, p.scale = kcache.shape[1], splits, 1.0 / hd ** 0.5
    scratch = torch.empty(max(1, n * nq * splits * (hd + 2)), dtype=torch.float32, device=dev)
    p.scratch = scratch.data_ptr()
    L.check(L.lib().b2_attn_rows(C.byref(p), C.c_void_p(seq_rows.data_ptr()), seq_rows.shape[0] - 1, hd, L.stream()),
            "attn_rows")
    return out


def attn_prefill_tc(q, rows_meta, kcache, vcache, nq, nkv, hd, gate_off=-1, row_base=0, n_rows_seq=None, out=None):
    """Causal attention of one sequence's prompt rows on the tcgen05 tensor cores (csrc/attention_tc.cu).
    Rows [row_base, row_base + n_rows_seq) are in position order and carry no draft-tree masks."""
    n = q.shape[0]
    dev = q.device
    if out is None:
        out = torch.zeros(n, nq * hd, dtype=torch.float16, device=dev)
    if n_rows_seq is None:
        n_rows_seq = n - row_base
    st = _tc_status.get(dev)
    if st is None:
        st = _tc_status[dev] = torch.zeros(64, dtype=torch.int32, device=dev)
    p = L.AttnParams()
    p.q, p.ldq, p.gate_off = q.data_ptr(), q.stride(0), gate_off
    p.kcache, p.vcache, p.rows = kcache.data_ptr(), vcache.data_ptr(), rows_meta.data_ptr()
    p.out, p.ldo, p.n_rows, p.nq, p.nkv = out.data_ptr(), out.stride(0), n, nq, nkv
    p.max_seq, p.splits, p.scale = kcache.shape[1], 1, 1.0 / hd ** 0.5
    L.check(L.lib().b2_attn_prefill_tc(C.byref(p), row_base, n_rows_seq, kcache.shape[0], hd,
                                       C.c_void_p(st.data_ptr()), L.stream()), "attn_prefill_tc")
    return out


def deltanet_step(proj, offs, conv_w, conv_state, state, A_log, dt_bias, norm_w, rows_meta, seq_rows, nk, nv,
                  dk, dv, xn=None, wa=None, wb=None, out=None, commit=True, eps=1e-6, ln=None):
    """offs = (off_q, off_k, off_v, off_z, off_a, off_b)."""
    n = proj.shape[0]
    if out is None:
        out = torch.empty(n, nv * dv, dtype=torch.float16, device=proj.device)
    p = L.DeltaParams()
    p.proj, p.ld = proj.data_ptr(), proj.stride(0)
    p.off_q, p.off_k, p.off_v, p.off_z, p.off_a, p.off_b = offs
    if xn is not None:
        p.xn, p.ldx, p.H = xn.data_ptr(), xn.stride(0), xn.shape[1]
        p.wa, p.wb = wa.data_ptr(), wb.data_ptr()
    if ln is not None:
        p.ln, p.H = ln, ln.H
        p.wa, p.wb = wa.data_ptr(), wb.data_ptr()
    p.conv_w, p.conv_state, p.state = conv_w.data_ptr(), conv_state.data_ptr(), state.data_ptr()
    p.A_log, p.dt_bias, p.norm_w = A_log.data_ptr(), dt_bias.data_ptr(), norm_w.data_ptr()
    p.seq_rows, p.rows, p.out, p.ldo = seq_rows.data_ptr(), rows_meta.data_ptr(), out.data_ptr(), out.stride(0)
    p.nk, p.nv, p.n_seqs, p.eps, p.commit = nk, nv, seq_rows.shape[0] - 1, eps, 1 if commit else 0
    L.check(L.lib().b2_deltanet_step(C.byref(p), dk, dv, L.stream()), "deltanet_step")
    return out


def ab_proj(x, wa, wb):
    """[rows, 2*nv] fp16: a = x @ wa^T, b = x @ wb^T (the DeltaNet gate projections)."""
    rows, H = x.shape
    nv = wa.shape[0]
    ab = torch.empty(rows, 2 * nv, dtype=torch.float16, device=x.device)
    L.check(L.lib().b2_ab_proj(_vp(x), x.stride(0), _vp(wa), _vp(wb), nv, H, _vp(ab), ab.stride(0), rows, L.stream()),
            "ab_proj")
    return ab


def deltanet_chunk(proj, offs, ab, conv_w, conv_state, state, A_log, dt_bias, norm_w, rows_meta, seq_rows, nk, nv,
                   dk, dv, out=None, commit=True, eps=1e-6, prepass: int = 0):
    """Chunked scan over each sequence's rows; ab: fp16 [rows, >= 2*nv] with a | b.  prepass (one sequence):
    1 = the q / k convolution and norms run once in a parallel kernel instead of inside the scan; 2 = also the
    state-independent products of every chunk and the inverse of its triangle."""
    n = proj.shape[0]
    if out is None:
        out = torch.empty(n, nv * dv, dtype=torch.float16, device=proj.device)
    p = L.DeltaParams()
    p.proj, p.ld = proj.data_ptr(), proj.stride(0)
    p.off_q, p.off_k, p.off_v, p.off_z, p.off_a, p.off_b = offs
    p.conv_w, p.conv_state, p.state = conv_w.data_ptr(), conv_state.data_ptr(), state.data_ptr()
    p.A_log, p.dt_bias, p.norm_w = A_log.data_ptr(), dt_bias.data_ptr(), norm_w.data_ptr()
    p.seq_rows, p.rows, p.out, p.ldo = seq_rows.data_ptr(), rows_meta.data_ptr(), out.data_ptr(), out.stride(0)
    p.nk, p.nv, p.n_seqs, p.eps, p.commit = nk, nv, seq_rows.shape[0] - 1, eps, 1 if commit else 0
    qk = torch.empty(n, 2 * nk * dk, dtype=torch.float16, device=proj.device) if prepass else None
    L.lib().b2_deltanet_tw_floats.restype = C.c_longlong
    tw = torch.empty(int(L.lib().b2_deltanet_tw_floats(nv, n)), dtype=torch.float32, device=proj.device) if int(prepass) > 1 else None
    L.check(L.lib().b2_deltanet_chunk(C.byref(p), _vp(ab), ab.stride(0), _vp(qk) if qk is not None else None,
                                      2 * nk * dk, n, _vp(tw) if tw is not None else None, dk, dv, L.stream()), "deltanet_chunk")
    return out


def argmax(logits: torch.Tensor, vocab_offset: int = 0, blocks: int = 16, comm: Optional[L.CommCtx] = None):
    n, V = logits.shape
    dev = logits.device
    out = torch.empty(n, dtype=torch.int32, device=dev)
    p = L.ArgmaxParams()
    p.logits, p.ld, p.n_rows, p.vocab_local, p.vocab_offset, p.blocks = logits.data_ptr(), logits.stride(0), n, V, vocab_offset, blocks
    scratch = torch.empty(n * blocks * 2, dtype=torch.float32, device=dev)
    counters = torch.zeros(n + 2, dtype=torch.int32, device=dev)
    p.scratch, p.counters, p.out_tokens = scratch.data_ptr(), counters.data_ptr(), out.data_ptr()
    p.comm = comm if comm is not None else L.null_comm()
    L.check(L.lib().b2_argmax(C.byref(p), L.stream()), "argmax")
    return out


def silu_mul(gate, up):
    out = torch.empty_like(gate)
    L.check(L.lib().b2_silu_mul(_vp(gate), _vp(up), _vp(out), C.c_size_t(gate.numel()), L.stream()), "silu_mul")
    return out


def sigmoid_mul_(x, gate):
    L.check(L.lib().b2_sigmoid_mul(_vp(x), _vp(gate), C.c_size_t(x.numel()), L.stream()), "sigmoid_mul")
    return x


def residual_add_(h, delta):
    d32 = delta if delta.dtype == torch.float32 else None
    d16 = delta if delta.dtype == torch.float16 else None
    L.check(L.lib().b2_residual_add(_vp(h), _vp(d32), _vp(d16), C.c_size_t(h.numel()), L.stream()), "residual_add")
    return h


_tc_status = {}


def sample_top_p(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 50, top_p: float = 0.9,
                 repetition_penalty: float = 1.0, past: Optional[torch.Tensor] = None,
                 n_past: Optional[torch.Tensor] = None, seed: int = 0, vocab_offset: int = 0, debug: bool = False,
                 comm: Optional[L.CommCtx] = None, vocab_total: int = 0):
    """Sample one token per row of fp32 logits [rows, vocab] on the device (temperature > 0).
    `past`: int32 [rows, max_past] token ids for the repetition penalty with counts `n_past`.
    The logits are modified in place by the penalty.  Returns int32 [rows] (and, with `debug`,
    the kept candidate ids and their probabilities, [rows, 1024] each).  With `comm` (tensor parallel,
    one row): `logits` is this rank's vocabulary slice starting at `vocab_offset`; the ranks exchange their
    candidate lists through symmetric memory inside the kernel and all return the same token."""
    n, V = logits.shape
    dev = logits.device
    out = torch.empty(n, dtype=torch.int32, device=dev)
    p = L.SampleParams()
    p.logits, p.ld, p.n_rows, p.vocab, p.vocab_offset = logits.data_ptr(), logits.stride(0), n, V, vocab_offset
    p.temperature, p.top_p, p.rep_penalty, p.top_k = temperature, top_p, repetition_penalty, top_k
    if past is not None:
        p.past, p.n_past, p.max_past = past.data_ptr(), n_past.data_ptr(), past.shape[1]
    p.seed, p.out_tokens = seed & 0xFFFFFFFFFFFFFFFF, out.data_ptr()
    p.comm = comm if comm is not None else L.null_comm()
    p.vocab_total = vocab_total
    ids = probs = None
    if debug:
        ids = torch.empty(n, L.SAMPLE_MAX_CAND, dtype=torch.int32, device=dev)
        probs = torch.empty(n, L.SAMPLE_MAX_CAND, dtype=torch.float32, device=dev)
        p.dbg_ids, p.dbg_probs = ids.data_ptr(), probs.data_ptr()
    L.check(L.lib().b2_sample(C.byref(p), L.stream()), "sample")
    return (out, ids, probs) if debug else out


def gemm_int4_tc(pk, x: torch.Tensor, out: torch.Tensor, epi: int = L.TC_EPI_STORE_F16,
                 t_tile: Optional[int] = None, n_valid: Optional[int] = None, k_splits: int = 1, m_halves: int = 1,
                 cta_pair: bool = False):
    """out[t][n] (epi) = x[t, :K] @ W for a PackedInt4 matrix on the tcgen05 tensor cores.
    x: fp16 [T, K] (row stride multiple of 8).  SILU_PAIR: out[t][j] = silu(gate_j) * up_j for
    the gate/up-interleaved matrix; RESID_F32: out (fp32) += product, optionally from k_splits CTAs
    per output tile that add their partial products atomically.  m_halves = 2: 256-output tiles (t_tile <= 256,
    padded N a multiple of 256; otherwise the launcher falls back to 128-output tiles)."""
    T = x.shape[0]
    dev = x.device
    if t_tile is None:
        t_tile = min(512, -(-T // 16) * 16)
    st = _tc_status.get(dev)
    if st is None:
        st = _tc_status[dev] = torch.zeros(64, dtype=torch.int32, device=dev)
    p = L.GemmTcParams()
    p.qfrag, p.szfrag = pk.qfrag.data_ptr(), pk.szfrag.data_ptr()
    p.K, p.KB, p.NTL, p.G, p.off32, p.gshift = pk.K, pk.KB, pk.NTL, pk.G, pk.off32, pk.gshift
    if m_halves == 2:
        t_tile = min(t_tile, 256)
    p.T, p.t_tile, p.epi, p.k_splits, p.m_halves, p.cta_pair = T, t_tile, epi, k_splits, m_halves, int(cta_pair)
    if n_valid is None:
        n_valid = pk.n_pad // 2 if epi == L.TC_EPI_SILU_PAIR else pk.N
    p.n_valid, p.ldo, p.out, p.status = n_valid, out.stride(0), out.data_ptr(), st.data_ptr()
    L.check(L.lib().b2_gemm_int4_tc(C.byref(p), C.c_void_p(x.data_ptr()), x.stride(0), L.stream()), "gemm_int4_tc")
    return out


def gemm_f16_tc(w: torch.Tensor, x: torch.Tensor, out: torch.Tensor, epi: int = L.TC_EPI_STORE_F32,
                t_tile: Optional[int] = None):
    """out[t][n] (epi) = x[t, :K] @ w[n, :K] for dense fp16 weights on the tcgen05 tensor cores
    (the lm_head of many rows).  K must be a multiple of 64."""
    T, dev = x.shape[0], x.device
    if t_tile is None:
        t_tile = min(512, -(-T // 16) * 16)
    st = _tc_status.get(dev)
    if st is None:
        st = _tc_status[dev] = torch.zeros(64, dtype=torch.int32, device=dev)
    p = L.GemmTcParams()
    p.K, p.T, p.t_tile, p.epi = w.shape[1], T, t_tile, epi
    p.n_valid, p.ldo, p.out, p.status = w.shape[0], out.stride(0), out.data_ptr(), st.data_ptr()
    L.check(L.lib().b2_gemm_f16_tc(C.byref(p), C.c_void_p(w.data_ptr()), w.stride(0), C.c_void_p(x.data_ptr()),
                                   x.stride(0), L.stream()), "gemm_f16_tc")
    return out


def gemm_tc_check_status(device=None):
    """Raise if a tcgen05 GEMM gave up on a bounded barrier wait since the last check."""
    for dev, st in _tc_status.items():
        if int(st[0].item()) != 0:
            st.zero_()
            raise RuntimeError("gemm_int4_tc: a bounded mbarrier wait expired")


def act_quant_int8(x: torch.Tensor):
    """Dynamic symmetric int8 quantisation of fp16 activations, one scale per row
    (reference: src/kernels/activation_quant.hip quantises per tensor; with one row the two agree).
    x: fp16 [T, K] with contiguous rows.  Returns (xq int8 [T, K], scale fp32 [T])."""
    assert x.dtype == torch.float16 and x.dim() == 2 and x.stride(1) == 1
    T, Kd = x.shape
    xq = torch.empty(T, Kd, dtype=torch.int8, device=x.device)
    scale = torch.empty(T, dtype=torch.float32, device=x.device)
    p = L.ActQuantParams()
    p.x, p.xq, p.scale, p.T, p.K, p.ldx = x.data_ptr(), xq.data_ptr(), scale.data_ptr(), T, Kd, x.stride(0)
    L.check(L.lib().b2_act_quant(C.byref(p), L.stream()), "act_quant")
    return xq, scale


def _linear_q8(w, xq, x_scale, N, out_dtype, w_scale=None, g_scale=None, group=0):
    T, Kd = xq.shape
    assert xq.dtype == torch.int8 and xq.is_contiguous() and x_scale.dtype == torch.float32 and w.is_contiguous()
    out = torch.empty(T, N, dtype=out_dtype, device=xq.device)
    p = L.Quant8Params()
    p.w, p.xq, p.x_scale, p.out = w.data_ptr(), xq.data_ptr(), x_scale.data_ptr(), out.data_ptr()
    p.w_scale, p.g_scale = _vp(w_scale), _vp(g_scale)
    p.K, p.N, p.T, p.ldo, p.group = Kd, N, T, N, group
    p.out_f16, p.w4 = int(out_dtype == torch.float16), int(g_scale is not None)
    L.check(L.lib().b2_linear_q8(C.byref(p), L.stream()), "linear_q8")
    return out


def linear_w8a8(w_int8: torch.Tensor, w_scale: torch.Tensor, xq: torch.Tensor, x_scale: torch.Tensor,
                out_dtype=torch.float32) -> torch.Tensor:
    """out[t][n] = x_scale[t] * w_scale[n] * sum_k xq[t][k] * w_int8[n][k] on the int8 tensor-core path
    (reference: src/kernels/gemv_w8a8.hip for one row, src/kernels/gemm_w8a8.hip for many).
    w_int8: [N, K] with K a multiple of 64; any number of rows."""
    assert w_int8.dtype == torch.int8 and w_scale.dtype == torch.float32
    return _linear_q8(w_int8, xq, x_scale, w_int8.shape[0], out_dtype, w_scale=w_scale)


def linear_w4a8(w_packed: torch.Tensor, g_scale: torch.Tensor, xq: torch.Tensor, x_scale: torch.Tensor,
                group: int = 128, out_dtype=torch.float32) -> torch.Tensor:
    """Same product for signed-nibble weights [N, K/8] int32 with per-group fp16 scales [K/group, N]
    (the layout `utils.quant.int4_to_w4a8` produces; reference: src/kernels/gemv_w4a8.hip).
    Integer accumulation inside a group, fp32 across groups."""
    assert w_packed.dtype == torch.int32 and g_scale.dtype == torch.float16 and g_scale.is_contiguous()
    return _linear_q8(w_packed, xq, x_scale, w_packed.shape[0], out_dtype, g_scale=g_scale, group=group)


# -- probes (csrc/comm.cu; reference: src/kernels/p2p_bandwidth_kernels.hip:187-278) ------------------

def probe_read(src_ptr: int, nbytes: int, dst_ptr: Optional[int] = None, multimem: bool = False, ctas: int = 296):
    """Stream `nbytes` (a multiple of 16) from a device address -- local memory, a peer's mapping, or (with
    `multimem`) a multicast address read with multimem.ld_reduce -- into registers, or into `dst_ptr`
    (local or peer) when given.  Launches on the current stream; time it with CUDA events."""
    L.check(L.lib().b2_probe_read(C.c_void_p(src_ptr), None if dst_ptr is None else C.c_void_p(dst_ptr),
                                  C.c_size_t(nbytes), int(multimem), ctas, L.stream()), "probe_read")


def probe_latency(chain: torch.Tensor, hops: int, chain_ptr: Optional[int] = None) -> float:
    """Average latency (ns) of `hops` dependent 4-byte loads that walk the index chain stored in `chain`
    (uint32 indices; `chain_ptr` overrides the address, e.g. with a peer's mapping of the same buffer)."""
    out = torch.zeros(2, dtype=torch.int64, device=chain.device)
    L.check(L.lib().b2_probe_latency(C.c_void_p(chain_ptr if chain_ptr is not None else chain.data_ptr()), hops,
                                     C.c_void_p(out.data_ptr()), L.stream()), "probe_latency")
    torch.cuda.synchronize(chain.device)
    return float(out[0].item()) / hops


def wait_self_test(wait_us: int = 2000) -> dict:
    """Run the bounded device wait on a flag that nothing sets and return the status record it leaves
    ({code, kernel, peer, epoch}): the wait must give up after `wait_us` and the context must stay usable."""
    dev = torch.device("cuda", torch.cuda.current_device())
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    c = L.null_comm()
    c.status, c.wait_ns = status.data_ptr(), int(wait_us) * 1000
    L.check(L.lib().b2_wait_test(C.byref(c), C.c_void_p(flag.data_ptr()), L.stream()), "wait_test")
    torch.cuda.synchronize(dev)
    st = status.tolist()
    return {"code": st[0], "kernel": st[1], "peer": st[2], "epoch": st[3]}
