"""Library baseline: the same model on PyTorch + cuBLAS + NCCL.

This is what the hand-written engine is measured against on the same GPUs: fp16
dense weights (INT4 checkpoints are dequantised at load), `F.linear` (cuBLAS) for
every projection, PyTorch's scaled-dot-product attention, the Gated DeltaNet
recurrence and its chunked form written with torch ops, `dist.all_reduce` (NCCL)
after the row-parallel projections, and an optional CUDA-graph capture of the
decode step (torch.cuda.graphs) so that the comparison is not about Python
overhead.  None of this package's CUDA kernels are used here.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

from ..config import QwenConfig
from ..models.weights import ModelWeights
from ..parallel.sharding import make_shard_spec

G_CLAMP = -20.0


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


class _Layer:
    pass


class TorchBaselineEngine:
    def __init__(self, cfg: QwenConfig, device=None, max_seq_len: int = 2048, tp_size: int = 1, tp_rank: int = 0,
                 dtype=torch.float16):
        self.cfg, self.dtype = cfg, dtype
        self.dev = torch.device(device if device is not None else "cuda")
        self.sp = make_shard_spec(cfg, tp_size, tp_rank)
        self.tp, self.rank, self.max_seq = tp_size, tp_rank, max_seq_len
        self.layers: List[_Layer] = []
        half = cfg.rotary_dim // 2
        freqs = 1.0 / (cfg.rope_theta ** (torch.arange(half, dtype=torch.float64) * 2.0 / cfg.rotary_dim))
        ang = torch.arange(max_seq_len, dtype=torch.float64)[:, None] * freqs[None, :]
        self.cos, self.sin = torch.cos(ang).float().to(self.dev), torch.sin(ang).float().to(self.dev)
        self.pos = torch.zeros(1, dtype=torch.long, device=self.dev)          # committed length (device, graph-safe)
        self.tok = torch.zeros(1, dtype=torch.long, device=self.dev)          # next input token
        self._graph = None
        self.launch_note = "library kernels (cuBLAS GEMV/GEMM, SDPA, elementwise, NCCL)"

    # ------------------------------------------------------------------ weights
    def _alloc_state(self):
        cfg, sp, dev = self.cfg, self.sp, self.dev
        for i, L in enumerate(self.layers):
            if L.full:
                L.k = torch.zeros(self.max_seq, sp.n_kv, cfg.head_dim, dtype=self.dtype, device=dev)
                L.v = torch.zeros_like(L.k)
            else:
                cd = 2 * sp.n_la_k * cfg.linear_key_head_dim + sp.n_la_v * cfg.linear_value_head_dim
                L.S = torch.zeros(sp.n_la_v, cfg.linear_key_head_dim, cfg.linear_value_head_dim, dtype=torch.float32, device=dev)
                L.conv = torch.zeros(cd, cfg.linear_conv_kernel_dim - 1, dtype=torch.float32, device=dev)

    def init_random(self, seed: int = 0):
        cfg, sp, dev, dt = self.cfg, self.sp, self.dev, self.dtype
        g = torch.Generator(device=dev)
        g.manual_seed(seed + 1000 * self.rank)
        H = cfg.hidden_size
        rnd = lambda n, k: (torch.randn(n, k, device=dev, generator=g) * 0.02).to(dt)
        ones = lambda n: torch.ones(n, dtype=dt, device=dev)
        for i in range(cfg.num_hidden_layers):
            L = _Layer()
            L.full = cfg.is_full_attention(i)
            L.attn_norm, L.ffn_norm = ones(H), ones(H)
            if L.full:
                qd, kvd = sp.n_q * cfg.head_dim, sp.n_kv * cfg.head_dim
                L.in_proj, L.out_proj = rnd(2 * qd + 2 * kvd, H), rnd(H, qd)
                L.q_norm, L.k_norm = ones(cfg.head_dim), ones(cfg.head_dim)
            else:
                kd, vd = sp.n_la_k * cfg.linear_key_head_dim, sp.n_la_v * cfg.linear_value_head_dim
                L.in_proj, L.out_proj = rnd(2 * kd + 2 * vd + 2 * sp.n_la_v, H), rnd(H, vd)
                L.conv_w = (torch.randn(2 * kd + vd, cfg.linear_conv_kernel_dim, device=dev, generator=g) * 0.3).float()
                L.A_log = (torch.rand(sp.n_la_v, device=dev, generator=g) * 1.5 - 1.0).float()
                L.dt_bias = (torch.randn(sp.n_la_v, device=dev, generator=g) * 0.5).float()
                L.la_norm = ones(cfg.linear_value_head_dim)
            L.gate_up, L.down = rnd(2 * sp.ffn_local, H), rnd(H, sp.ffn_local)
            self.layers.append(L)
        g2 = torch.Generator(device=dev)
        g2.manual_seed(seed + 7)
        self.embed = (torch.randn(cfg.vocab_size, H, device=dev, generator=g2) * 0.05).to(dt)
        self.lm_head = (torch.randn(sp.vocab_local, H, device=dev, generator=g) * 0.05).to(dt)
        self.final_norm = ones(H)
        self._alloc_state()

    def load_model(self, mw: ModelWeights):
        """`mw`: this rank's shard in engine format; INT4 projections are dequantised."""
        dev, dt = self.dev, self.dtype
        d = lambda lin: lin.dense(torch.float32).to(device=dev, dtype=dt)
        for lw in mw.layers:
            L = _Layer()
            L.full = lw.is_full
            L.attn_norm, L.ffn_norm = lw.attn_norm.to(dev, dt), lw.ffn_norm.to(dev, dt)
            if L.full:
                L.in_proj = torch.cat([d(lw.q), d(lw.q_gate), d(lw.k), d(lw.v)], 0)
                L.out_proj = d(lw.o)
                L.q_norm, L.k_norm = lw.q_norm.to(dev, dt), lw.k_norm.to(dev, dt)
            else:
                L.in_proj = torch.cat([d(lw.la_qkv), d(lw.la_z), d(lw.la_a), d(lw.la_b)], 0)
                L.out_proj = d(lw.la_out)
                L.conv_w = lw.la_conv1d.to(dev).float()
                L.A_log, L.dt_bias = lw.la_A_log.to(dev).float(), lw.la_dt_bias.to(dev).float()
                L.la_norm = lw.la_norm.to(dev, dt)
            L.gate_up, L.down = torch.cat([d(lw.gate), d(lw.up)], 0), d(lw.down)
            self.layers.append(L)
        self.embed, self.lm_head = mw.embed.to(dev, dt), mw.lm_head.to(dev, dt)
        self.final_norm = mw.final_norm.to(dev, dt)
        self._alloc_state()

    def reset(self):
        self.pos.zero_()
        for L in self.layers:
            if not L.full:
                L.S.zero_()
                L.conv.zero_()

    # ------------------------------------------------------------------ pieces
    def _all_reduce(self, x):
        if self.tp > 1:
            import torch.distributed as dist
            dist.all_reduce(x)
        return x

    def _rope(self, x, positions):
        """x[S, heads, hd]; interleaved or half-split partial rotation."""
        half = self.cfg.rotary_dim // 2
        rot = 2 * half
        c, s = self.cos[positions][:, None, :], self.sin[positions][:, None, :]
        xf = x.float()
        out = xf.clone()
        if self.cfg.rope_style == "interleaved":
            x0, x1 = xf[..., 0:rot:2], xf[..., 1:rot:2]
            out[..., 0:rot:2] = x0 * c - x1 * s
            out[..., 1:rot:2] = x0 * s + x1 * c
        else:
            x0, x1 = xf[..., :half], xf[..., half:rot]
            out[..., :half] = x0 * c - x1 * s
            out[..., half:rot] = x0 * s + x1 * c
        return out.to(x.dtype)

    def _full_attention(self, L, xn, positions, decode: bool):
        cfg, sp = self.cfg, self.sp
        S, hd = xn.shape[0], cfg.head_dim
        qd, kvd = sp.n_q * hd, sp.n_kv * hd
        p = F.linear(xn, L.in_proj)
        q, gate = p[:, :qd].view(S, sp.n_q, hd), p[:, qd:2 * qd].view(S, sp.n_q, hd)
        k, v = p[:, 2 * qd:2 * qd + kvd].view(S, sp.n_kv, hd), p[:, 2 * qd + kvd:].view(S, sp.n_kv, hd)
        q = self._rope(_rms(q, L.q_norm, cfg.rms_norm_eps), positions)
        k = self._rope(_rms(k, L.k_norm, cfg.rms_norm_eps), positions)
        L.k.index_copy_(0, positions, k)
        L.v.index_copy_(0, positions, v)
        if decode:
            # static shapes (graph-safe): attend over the whole cache with a length mask
            T = self.max_seq
            mask = (torch.arange(T, device=self.dev)[None, :] <= positions[:, None])[None]     # [1,S,T]
            K, V = L.k, L.v
        else:
            T = int(positions[-1].item()) + 1
            mask = (torch.arange(T, device=self.dev)[None, :] <= positions[:, None])[None]
            K, V = L.k[:T], L.v[:T]
        o = F.scaled_dot_product_attention(q.transpose(0, 1)[None], K.transpose(0, 1)[None], V.transpose(0, 1)[None],
                                           attn_mask=mask[None], enable_gqa=True)
        o = o[0].transpose(0, 1)
        if cfg.attn_output_gate:
            o = o * torch.sigmoid(gate.float()).to(o.dtype)
        return F.linear(o.reshape(S, qd), L.out_proj)

    def _deltanet(self, L, xn):
        cfg, sp = self.cfg, self.sp
        S = xn.shape[0]
        dk, dv, nk, nv = cfg.linear_key_head_dim, cfg.linear_value_head_dim, sp.n_la_k, sp.n_la_v
        kd, vd = nk * dk, nv * dv
        p = F.linear(xn, L.in_proj)
        qkv, z = p[:, :2 * kd + vd].float(), p[:, 2 * kd + vd:2 * kd + 2 * vd].view(S, nv, dv).float()
        a, b = p[:, 2 * kd + 2 * vd:2 * kd + 2 * vd + nv].float(), p[:, 2 * kd + 2 * vd + nv:].float()
        g = (-torch.exp(L.A_log) * F.softplus(a + L.dt_bias)).clamp(G_CLAMP, 0.0)
        beta = torch.sigmoid(b)
        full = torch.cat([L.conv.t(), qkv], 0)                               # [3+S, C]
        kw = L.conv_w.shape[1]
        c = sum(full[j:j + S] * L.conv_w[:, j][None, :] for j in range(kw))
        L.conv.copy_(full[-(kw - 1):].t())
        c = F.silu(c)
        l2 = lambda x: x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)
        q = l2(c[:, :kd].view(S, nk, dk)) / math.sqrt(dk)
        k = l2(c[:, kd:2 * kd].view(S, nk, dk))
        v = c[:, 2 * kd:].view(S, nv, dv)
        rep = nv // nk
        q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
        y = self._delta_recurrent(q, k, v, g, beta, L.S) if S < 16 else self._delta_chunked(q, k, v, g, beta, L.S)
        yn = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + 1e-6) * L.la_norm.float() * F.silu(z)
        return F.linear(yn.reshape(S, vd).to(self.dtype), L.out_proj)

    @staticmethod
    def _delta_recurrent(q, k, v, g, beta, state):
        ys = []
        for t in range(q.shape[0]):
            state.mul_(torch.exp(g[t])[:, None, None])
            mem = torch.einsum("hkv,hk->hv", state, k[t])
            delta = (v[t] - mem) * beta[t][:, None]
            state.add_(k[t][:, :, None] * delta[:, None, :])
            ys.append(torch.einsum("hkv,hk->hv", state, q[t]))
        return torch.stack(ys)

    @staticmethod
    def _delta_chunked(q, k, v, g, beta, state, chunk: int = 64):
        S, H, _ = q.shape
        dev = q.device
        ys = []
        for c0 in range(0, S, chunk):
            c1 = min(S, c0 + chunk)
            C = c1 - c0
            qc, kc, vc = (t[c0:c1].transpose(0, 1) for t in (q, k, v))
            gc, bc = g[c0:c1].t(), beta[c0:c1].t()
            G = torch.cumsum(gc, 1)
            diff = G[:, :, None] - G[:, None, :]
            lower = torch.tril(torch.ones(C, C, dtype=torch.bool, device=dev), -1)
            lower_eq = torch.tril(torch.ones(C, C, dtype=torch.bool, device=dev))
            decay = torch.exp(diff.masked_fill(~lower_eq, 0.0))
            A = (bc[:, :, None] * decay * (kc @ kc.transpose(1, 2))).masked_fill(~lower, 0.0)
            eye = torch.eye(C, device=dev).expand(H, C, C)
            T = torch.linalg.solve_triangular(eye + A, eye, upper=False, unitriangular=True)
            eg = torch.exp(G)
            U = T @ (bc[:, :, None] * vc) - T @ ((bc * eg)[:, :, None] * kc) @ state
            W = (decay * (qc @ kc.transpose(1, 2))).masked_fill(~lower_eq, 0.0)
            Y = eg[:, :, None] * (qc @ state) + W @ U
            tail = torch.exp(G[:, -1:] - G)
            state.copy_(eg[:, -1][:, None, None] * state + (tail[:, :, None] * kc).transpose(1, 2) @ U)
            ys.append(Y.transpose(0, 1))
        return torch.cat(ys)

    # ------------------------------------------------------------------ forward
    def _forward(self, tokens: torch.Tensor, positions: torch.Tensor, decode: bool):
        cfg = self.cfg
        x = self.embed[tokens]
        F_loc = self.sp.ffn_local
        for L in self.layers:
            xn = _rms(x, L.attn_norm, cfg.rms_norm_eps)
            p = self._full_attention(L, xn, positions, decode) if L.full else self._deltanet(L, xn)
            x = x + self._all_reduce(p)
            xn = _rms(x, L.ffn_norm, cfg.rms_norm_eps)
            gu = F.linear(xn, L.gate_up)
            f = F.linear(F.silu(gu[:, :F_loc]) * gu[:, F_loc:], L.down)
            x = x + self._all_reduce(f)
        return _rms(x, self.final_norm, cfg.rms_norm_eps)

    def _next_token(self, h_last: torch.Tensor) -> torch.Tensor:
        logits = F.linear(h_last, self.lm_head).float()                       # [1, vocab_local]
        if self.tp == 1:
            return torch.argmax(logits, -1)
        import torch.distributed as dist
        v, i = logits.max(-1)
        pair = torch.stack([v, (i + self.sp.vocab[0]).float()], -1)          # [1, 2]
        allp = [torch.empty_like(pair) for _ in range(self.tp)]
        dist.all_gather(allp, pair)
        allp = torch.stack(allp)                                              # [tp, 1, 2]
        best = torch.argmax(allp[:, :, 0], 0)
        return allp[best, torch.arange(1, device=self.dev), 1].long()

    @torch.no_grad()
    def prefill(self, tokens: Sequence[int]) -> int:
        self.reset()
        t = torch.as_tensor(list(tokens), dtype=torch.long, device=self.dev)
        positions = torch.arange(len(tokens), device=self.dev)
        h = self._forward(t, positions, decode=False)
        self.pos.fill_(len(tokens))
        self.tok.copy_(self._next_token(h[-1:]))
        return int(self.tok.item())

    @torch.no_grad()
    def _decode_once(self):
        h = self._forward(self.tok, self.pos, decode=True)
        self.tok.copy_(self._next_token(h))
        self.pos.add_(1)

    @torch.no_grad()
    def decode(self, n_steps: int, graph: bool = True, collect: bool = False) -> Optional[List[int]]:
        """n greedy steps; with `graph` the step is captured once into a CUDA graph and replayed."""
        out = []
        if graph and self._graph is None:
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                snap = [(L.S.clone(), L.conv.clone()) for L in self.layers if not L.full]
                pos0, tok0 = self.pos.clone(), self.tok.clone()
                for _ in range(2):
                    self._decode_once()                                      # warm up library workspaces
                for L, (S0, c0) in zip([L for L in self.layers if not L.full], snap):
                    L.S.copy_(S0); L.conv.copy_(c0)
                self.pos.copy_(pos0); self.tok.copy_(tok0)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._decode_once()
            for L, (S0, c0) in zip([L for L in self.layers if not L.full], snap):
                L.S.copy_(S0); L.conv.copy_(c0)
            self.pos.copy_(pos0); self.tok.copy_(tok0)
        for _ in range(n_steps):
            if graph:
                self._graph.replay()
            else:
                self._decode_once()
            if collect:
                out.append(int(self.tok.item()))
        return out if collect else None

    def weight_bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for L in self.layers for t in (L.in_proj, L.out_proj, L.gate_up, L.down))
        return n + self.lm_head.numel() * self.lm_head.element_size()
