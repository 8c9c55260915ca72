"""fp32 PyTorch reference of the hybrid decoder: the numerical oracle.

Every CUDA kernel and every engine mode in this package is tested against the
functions here.  The math follows the reference's decode path
(reference: src/inference/engine.py:1440-1501 for the layer skeleton,
:1943-2092 for gated full attention, :2094-2206 for the Gated DeltaNet step that
the reference itself uses as its CPU oracle) with all arithmetic in fp32 and no
fp16 rounding of intermediates.

`OracleEngine` also runs as one rank of a tensor-parallel job over any
`Communicator` (gloo on CPU), which is how the sharder, the three all-reduce
placements and TP=1 vs TP=2 agreement are tested without a GPU.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..config import QwenConfig
from ..parallel.comm import Communicator, SingleComm
from ..parallel.sharding import ShardSpec, make_shard_spec
from .weights import LayerWeights, ModelWeights

DELTA_EPS = 1e-6
G_CLAMP = -20.0


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * w.float()


def rope_tables(cfg: QwenConfig, positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin[len(positions), rotary_dim/2] with freq_i = theta^(-2i/rot)
    (reference: src/inference/engine.py:1025-1046)."""
    rot = cfg.rotary_dim
    half = rot // 2
    freqs = 1.0 / (cfg.rope_theta ** (torch.arange(half, dtype=torch.float64) * 2.0 / rot))
    ang = positions.to(torch.float64)[:, None] * freqs[None, :]
    return torch.cos(ang).float(), torch.sin(ang).float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, style: str) -> torch.Tensor:
    """x[S, H, hd]; rotates the first 2*cos.shape[1] dims of every head."""
    half = cos.shape[1]
    rot = 2 * half
    out = x.clone()
    c, s = cos[:, None, :], sin[:, None, :]
    if style == "interleaved":
        x0, x1 = x[..., 0:rot:2], x[..., 1:rot:2]
        out[..., 0:rot:2] = x0 * c - x1 * s
        out[..., 1:rot:2] = x0 * s + x1 * c
    else:
        x0, x1 = x[..., :half], x[..., half:rot]
        out[..., :half] = x0 * c - x1 * s
        out[..., half:rot] = x0 * s + x1 * c
    return out


def attention(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """q[S, Hq, hd], K/V[T, Hkv, hd], mask[S, T] bool (True = attend)."""
    S, Hq, hd = q.shape
    Hkv = K.shape[1]
    rep = Hq // Hkv
    Kx = K.repeat_interleave(rep, dim=1)
    Vx = V.repeat_interleave(rep, dim=1)
    sc = torch.einsum("shd,thd->hst", q, Kx) / math.sqrt(hd)
    sc = sc.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(sc, dim=-1)
    return torch.einsum("hst,thd->shd", p, Vx)


def causal_mask(S: int, ctx: int) -> torch.Tensor:
    """Query i (absolute position ctx+i) sees keys 0..ctx+i."""
    t = torch.arange(ctx + S)[None, :]
    return t <= (ctx + torch.arange(S))[:, None]


def tree_mask(parents: Sequence[int], ctx: int) -> torch.Tensor:
    """Mask [T, ctx+T]: every draft node sees the whole context, itself and its
    ancestors (reference: src/inference/tree_attention.py:186-208)."""
    T = len(parents)
    m = torch.zeros(T, ctx + T, dtype=torch.bool)
    m[:, :ctx] = True
    for i in range(T):
        j = i
        while j >= 0:
            m[i, ctx + j] = True
            j = parents[j]
    return m


# -- Gated DeltaNet ---------------------------------------------------------

def l2norm(x: torch.Tensor) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).sum(dim=-1, keepdim=True) + DELTA_EPS)


def deltanet_gates(a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor,
                   dt_bias: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """log-decay g (clamped to [-20, 0]) and beta = sigmoid(b), both [S, Hv]."""
    g = -torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float())
    return g.clamp(G_CLAMP, 0.0), torch.sigmoid(b.float())


def deltanet_recurrent(q, k, v, g, beta, state):
    """Token-serial gated delta rule.  q,k[S,H,dk] (already L2-normalised and q
    scaled), v[S,H,dv], g,beta[S,H], state[H,dk,dv] (updated in place).
    Returns y[S,H,dv]."""
    S = q.shape[0]
    ys = []
    for t in range(S):
        state *= torch.exp(g[t])[:, None, None]
        mem = torch.einsum("hkv,hk->hv", state, k[t])
        delta = (v[t] - mem) * beta[t][:, None]
        state += torch.einsum("hk,hv->hkv", k[t], delta)
        ys.append(torch.einsum("hkv,hk->hv", state, q[t]))
    return torch.stack(ys)


def deltanet_chunked(q, k, v, g, beta, state, chunk: int = 64):
    """Chunk-parallel form of the same recurrence (what the prefill kernel
    computes).  Within a chunk, with G the running sum of g from the chunk start:
        A[i,j] = beta_i exp(G_i-G_j) (k_i.k_j)  for j<i,  T = (I+A)^-1
        U = T (beta*V) - T (beta*exp(G)*K) S0
        Y = exp(G) Q S0 + tril(exp(G_i-G_j) (q_i.k_j)) U
        S' = exp(G_C) S0 + (exp(G_C-G) K)^T U
    """
    S, H, dk = q.shape
    ys = []
    for c0 in range(0, S, chunk):
        c1 = min(S, c0 + chunk)
        C = c1 - c0
        qc, kc, vc = (t[c0:c1].transpose(0, 1) for t in (q, k, v))      # [H,C,*]
        gc, bc = g[c0:c1].t(), beta[c0:c1].t()                          # [H,C]
        G = torch.cumsum(gc, dim=1)
        diff = G[:, :, None] - G[:, None, :]                            # G_i - G_j
        lower = torch.tril(torch.ones(C, C, dtype=torch.bool), -1)
        lower_eq = torch.tril(torch.ones(C, C, dtype=torch.bool))
        decay = torch.exp(diff.masked_fill(~lower_eq, 0.0))
        A = (bc[:, :, None] * decay * (kc @ kc.transpose(1, 2))).masked_fill(~lower, 0.0)
        eye = torch.eye(C).expand(H, C, C)
        T = torch.linalg.solve_triangular(eye + A, eye, upper=False, unitriangular=True)
        eg = torch.exp(G)
        U = T @ (bc[:, :, None] * vc) - T @ ((bc * eg)[:, :, None] * kc) @ state
        W = (decay * (qc @ kc.transpose(1, 2))).masked_fill(~lower_eq, 0.0)
        Y = eg[:, :, None] * (qc @ state) + W @ U
        tail = torch.exp(G[:, -1:] - G)                                  # [H,C]
        state.copy_(eg[:, -1][:, None, None] * state + (tail[:, :, None] * kc).transpose(1, 2) @ U)
        ys.append(Y.transpose(0, 1))
    return torch.cat(ys)


def causal_conv1d(x: torch.Tensor, conv_state: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Depthwise causal conv over [state | x] followed by SiLU.  x[S, C],
    conv_state[C, k-1] (oldest first; updated in place to the last k-1 inputs),
    w[C, k] (reference: src/inference/engine.py:2119-2136)."""
    S, C = x.shape
    k = w.shape[1]
    full = torch.cat([conv_state.t().float(), x.float()], dim=0)        # [k-1+S, C]
    out = torch.zeros(S, C)
    for j in range(k):
        out += full[j:j + S] * w[:, j].float()[None, :]
    conv_state.copy_(full[-(k - 1):].t())
    return F.silu(out)


def gated_rmsnorm(y: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float = DELTA_EPS):
    """y/rms(y) * w * silu(z) per head; plain w, no 1+w
    (reference: src/inference/engine.py:2188-2194)."""
    yn = y * torch.rsqrt(y.pow(2).mean(dim=-1, keepdim=True) + eps)
    return yn * w.float() * F.silu(z)


# -- engine -----------------------------------------------------------------

@dataclass
class OracleSeqState:
    """Everything position-dependent for one sequence: the explicit
    `SequenceState` the reference lacks (its speculative rollback only rewinds a
    length counter: src/inference/tp_engine.py:1673-1687)."""
    length: int = 0
    k: Dict[int, torch.Tensor] = field(default_factory=dict)
    v: Dict[int, torch.Tensor] = field(default_factory=dict)
    S: Dict[int, torch.Tensor] = field(default_factory=dict)
    conv: Dict[int, torch.Tensor] = field(default_factory=dict)

    def clone(self) -> "OracleSeqState":
        c = lambda d: {i: t.clone() for i, t in d.items()}
        return OracleSeqState(self.length, c(self.k), c(self.v), c(self.S), c(self.conv))


class OracleEngine:
    def __init__(self, weights: ModelWeights, tp_size: int = 1, tp_rank: int = 0,
                 comm: Optional[Communicator] = None, ar_mode: str = "exact",
                 max_seq_len: int = 2048, max_batch: int = 1, chunked_deltanet: bool = False):
        """`weights` must already be this rank's shard (parallel.sharding.shard_model)."""
        self.cfg = weights.config
        self.w = weights
        self.spec: ShardSpec = make_shard_spec(self.cfg, tp_size, tp_rank)
        self.comm = comm or SingleComm()
        self.ar_mode = ar_mode if tp_size > 1 else "exact"
        self.max_seq_len = max_seq_len
        self.chunked = chunked_deltanet
        self._dense: Dict[Tuple[int, str], torch.Tensor] = {}
        self.seqs: List[OracleSeqState] = [self._fresh() for _ in range(max_batch)]

    # -- state --------------------------------------------------------------
    def _fresh(self) -> OracleSeqState:
        cfg, sp = self.cfg, self.spec
        st = OracleSeqState()
        for i in range(cfg.num_hidden_layers):
            if cfg.is_full_attention(i):
                st.k[i] = torch.zeros(self.max_seq_len, sp.n_kv, cfg.head_dim)
                st.v[i] = torch.zeros(self.max_seq_len, sp.n_kv, cfg.head_dim)
            else:
                st.S[i] = torch.zeros(sp.n_la_v, cfg.linear_key_head_dim, cfg.linear_value_head_dim)
                cd = 2 * sp.n_la_k * cfg.linear_key_head_dim + sp.n_la_v * cfg.linear_value_head_dim
                st.conv[i] = torch.zeros(cd, cfg.linear_conv_kernel_dim - 1)
        return st

    def reset(self, seq: Optional[int] = None):
        for b in ([seq] if seq is not None else range(len(self.seqs))):
            self.seqs[b] = self._fresh()

    def snapshot(self, seq: int = 0) -> OracleSeqState:
        return self.seqs[seq].clone()

    def restore(self, snap: OracleSeqState, seq: int = 0):
        self.seqs[seq] = snap.clone()

    # -- pieces -------------------------------------------------------------
    def _lin(self, li: int, name: str, x: torch.Tensor) -> torch.Tensor:
        key = (li, name)
        if key not in self._dense:
            self._dense[key] = getattr(self.w.layers[li], name).dense(torch.float32)
        return x @ self._dense[key].t()

    def _full_attention(self, li, lw, xn, st, positions, mask, write_at):
        cfg, sp = self.cfg, self.spec
        S = xn.shape[0]
        hd = cfg.head_dim
        q = self._lin(li, "q", xn).view(S, sp.n_q, hd)
        gate = self._lin(li, "q_gate", xn).view(S, sp.n_q, hd)
        k = self._lin(li, "k", xn).view(S, sp.n_kv, hd)
        v = self._lin(li, "v", xn).view(S, sp.n_kv, hd)
        q = rmsnorm(q, lw.q_norm, cfg.rms_norm_eps)
        k = rmsnorm(k, lw.k_norm, cfg.rms_norm_eps)
        cos, sin = rope_tables(cfg, positions)
        q = apply_rope(q, cos, sin, cfg.rope_style)
        k = apply_rope(k, cos, sin, cfg.rope_style)
        st.k[li][write_at:write_at + S] = k
        st.v[li][write_at:write_at + S] = v
        T = mask.shape[1]
        o = attention(q, st.k[li][:T], st.v[li][:T], mask)
        if cfg.attn_output_gate:
            o = o * torch.sigmoid(gate)
        return self._lin(li, "o", o.reshape(S, sp.n_q * hd))

    def _linear_attention(self, li, lw, xn, st, parents=None):
        cfg, sp = self.cfg, self.spec
        S = xn.shape[0]
        dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        nk, nv = sp.n_la_k, sp.n_la_v
        qkv = self._lin(li, "la_qkv", xn)
        a = self._lin(li, "la_a", xn)
        b = self._lin(li, "la_b", xn)
        z = self._lin(li, "la_z", xn).view(S, nv, dv)
        g, beta = deltanet_gates(a, b, lw.la_A_log, lw.la_dt_bias)

        def run(x_qkv, g_, beta_, conv_state, state):
            c = causal_conv1d(x_qkv, conv_state, lw.la_conv1d)
            n = x_qkv.shape[0]
            q = l2norm(c[:, :nk * dk].reshape(n, nk, dk)) / math.sqrt(dk)
            k = l2norm(c[:, nk * dk:2 * nk * dk].reshape(n, nk, dk))
            v = c[:, 2 * nk * dk:].reshape(n, nv, dv)
            rep = nv // nk
            q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
            fn = deltanet_chunked if (self.chunked and n > 1) else deltanet_recurrent
            return fn(q, k, v, g_, beta_, state)

        if parents is None:
            y = run(qkv, g, beta, st.conv[li], st.S[li])
        else:
            # tree verify: every node continues from its parent's state; the
            # sequence state itself is left untouched (commit happens after
            # acceptance by re-running the accepted path).
            y = torch.zeros(S, nv, dv)
            node_state: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
            for i, p in enumerate(parents):
                cs, ss = (st.conv[li], st.S[li]) if p < 0 else node_state[p]
                cs, ss = cs.clone(), ss.clone()
                y[i] = run(qkv[i:i + 1], g[i:i + 1], beta[i:i + 1], cs, ss)[0]
                node_state[i] = (cs, ss)
        y = gated_rmsnorm(y, z, lw.la_norm)
        return self._lin(li, "la_out", y.reshape(S, nv * dv))

    def _ffn(self, li, xn):
        return self._lin(li, "down", F.silu(self._lin(li, "gate", xn)) * self._lin(li, "up", xn))

    # -- forward ------------------------------------------------------------
    def forward(self, embs: torch.Tensor, seq: int = 0, parents: Optional[Sequence[int]] = None,
                commit: bool = True) -> torch.Tensor:
        """Run S new tokens of sequence `seq` through every layer and return the
        residual stream [S, hidden] before the final norm.  With `parents`
        (draft tree, -1 = child of the last committed token) attention uses the
        tree mask, RoPE positions are length + depth, and nothing is committed."""
        cfg = self.cfg
        st = self.seqs[seq]
        x = embs.float().clone()
        S = x.shape[0]
        ctx = st.length
        if ctx + S > self.max_seq_len:
            raise ValueError("sequence exceeds max_seq_len")
        if parents is None:
            positions = ctx + torch.arange(S)
            mask = causal_mask(S, ctx)
        else:
            depth = []
            for i, p in enumerate(parents):
                depth.append(0 if p < 0 else depth[p] + 1)
            positions = ctx + torch.tensor(depth)
            mask = tree_mask(parents, ctx)
        tp = self.spec.tp_size > 1
        for li, lw in enumerate(self.w.layers):
            xn = rmsnorm(x, lw.attn_norm, cfg.rms_norm_eps)
            if lw.is_full:
                p = self._full_attention(li, lw, xn, st, positions, mask, ctx)
            else:
                p = self._linear_attention(li, lw, xn, st, parents)
            x_in = x
            if not tp or self.ar_mode == "exact":
                x = x + self.comm.all_reduce_sum(p)
            else:
                x = x + p                       # deferred: own partial only
            xn = rmsnorm(x, lw.ffn_norm, cfg.rms_norm_eps)
            f = self._ffn(li, xn)
            if tp and self.ar_mode == "deferred_consistent":
                x = x_in + self.comm.all_reduce_sum(p + f)
            else:
                x = x + self.comm.all_reduce_sum(f)
        if parents is None and commit:
            st.length = ctx + S
        return x

    # -- reference-compatible entry points ------------------------------------
    def prefill_step(self, embs: torch.Tensor, seq: int = 0) -> torch.Tensor:
        """Whole prompt in, hidden state of the last token out (final norm
        applied), like the reference (src/inference/engine.py:3009-3294)."""
        x = self.forward(embs, seq)
        return rmsnorm(x[-1], self.w.final_norm, self.cfg.rms_norm_eps)

    def decode_step(self, emb: torch.Tensor, position: Optional[int] = None, seq: int = 0):
        if position is not None and position != self.seqs[seq].length:
            raise ValueError("position must equal the current sequence length")
        x = self.forward(emb.reshape(1, -1), seq)
        return rmsnorm(x[0], self.w.final_norm, self.cfg.rms_norm_eps)

    def final_norm(self, x: torch.Tensor) -> torch.Tensor:
        return rmsnorm(x, self.w.final_norm, self.cfg.rms_norm_eps)

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """hidden (final-normed) -> fp32 logits over the full vocabulary; each
        rank multiplies its vocabulary slice and the slices are gathered."""
        local = hidden.float() @ self.w.lm_head.float().t()
        if self.spec.tp_size == 1:
            return local
        return torch.cat(self.comm.all_gather(local), dim=-1)

    def embed(self, token_ids) -> torch.Tensor:
        return self.w.embed[torch.as_tensor(token_ids, dtype=torch.long)].float()

    def score_tokens(self, tokens: Sequence[int], seq: int = 0) -> torch.Tensor:
        """log p(tokens[i+1] | tokens[:i+1]) for i = 0 .. n-2 (teacher forcing from an empty slot)."""
        self.reset(seq)
        x = self.forward(self.embed(list(tokens)), seq)
        logp = torch.log_softmax(self.compute_logits(self.final_norm(x)), dim=-1)
        nxt = torch.as_tensor(list(tokens)[1:], dtype=torch.long)
        return logp[:-1].gather(1, nxt[:, None])[:, 0]

    def perplexity(self, tokens: Sequence[int], seq: int = 0) -> float:
        return float(torch.exp(-self.score_tokens(tokens, seq).mean()))

    def greedy_generate(self, prompt_ids: Sequence[int], n_new: int, seq: int = 0):
        """Returns (tokens, logits per step)."""
        h = self.prefill_step(self.embed(list(prompt_ids)), seq)
        toks, logs = [], []
        for _ in range(n_new):
            logits = self.compute_logits(h)
            logs.append(logits)
            t = int(torch.argmax(logits))
            toks.append(t)
            h = self.decode_step(self.embed([t])[0], seq=seq)
        return toks, torch.stack(logs)
