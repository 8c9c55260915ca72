"""Single-GPU engine and per-rank worker of the tensor-parallel engine.

Same role and public surface as the reference's `InferenceEngine` (reference:
src/inference/engine.py:458-3785: embedding-in / hidden-out `decode_step`,
`prefill_step`, `compute_logits`, `load_layer_weights`, launch counters), built
differently:

* weights are packed into tensor-core fragment order and fused at load
  (Q|gate|K|V, q|k|v|z, gate/up interleaved) -- ops/packing.py;
* a C++ driver issues the whole step (csrc/driver.cu); the step reads positions
  and tokens from device memory, so ONE captured CUDA graph replays every token
  and `generate_tokens` can run many tokens without a host round trip;
* the token-level interface (`step_tokens`, `generate_tokens`) keeps embedding
  lookup, lm_head and arg-max on the device; the reference does those three on
  the host per token (reference: src/inference/generate.py:55-72,126-145);
* sequences have independent lengths; state can be snapshotted and restored.
"""
from __future__ import annotations

import ctypes as C
import logging
import os
import math
from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..config import EngineConfig, QwenConfig
from ..models.weights import LayerWeights, ModelWeights
from ..ops import lib as L
from ..ops.packing import (PackedInt4, concat_out, concat_out_dense, interleave_gate_up, launch_shape,
                           pack_int4, random_packed_int4)
from ..parallel.sharding import ShardSpec, make_shard_spec
from ..utils.quant import DenseLinear, Int4Linear
from .state import SequenceStates

log = logging.getLogger(__name__)
AR_MODE_ID = {"exact": 0, "deferred_ref": 1, "deferred_consistent": 2}


class DeviceLinear:
    """A projection resident on the GPU: packed INT4 or dense fp16 [N, K]."""

    def __init__(self, packed: Optional[PackedInt4] = None, dense: Optional[torch.Tensor] = None):
        self.packed, self.dense = packed, dense
        if dense is not None:
            self.N, self.K = dense.shape
            ctas_n = -(-self.N // 128)
            ks = 1 if ctas_n >= 148 else max(1, min(296 // ctas_n, self.K // 512))
            self.kslice = min(8192, -(-(-(-self.K // ks)) // 256) * 256)
            self.k_splits = -(-self.K // self.kslice)
        else:
            self.N, self.K = packed.N, packed.K

    @property
    def n_pad(self) -> int:
        return self.packed.n_pad if self.packed is not None else -(-self.N // 128) * 128

    def scratch_floats(self, rows: int) -> int:
        ks = self.packed.k_splits if self.packed is not None else self.k_splits
        return ks * rows * self.n_pad if ks > 1 else 0

    def desc(self) -> L.LinearDesc:
        d = L.LinearDesc()
        if self.packed is not None:
            p = self.packed
            d.kind, d.K, d.N, d.KB, d.NTL, d.G = L.LIN_INT4, p.K, p.N, p.KB, p.NTL, p.G
            d.off32, d.gshift, d.k_splits, d.L = p.off32, p.gshift, p.k_splits, p.L
            d.w, d.sz = p.qfrag.data_ptr(), p.szfrag.data_ptr()
        else:
            d.kind, d.K, d.N = L.LIN_F16, self.K, self.N
            d.ldw, d.kslice, d.k_splits = self.dense.stride(0), self.kslice, self.k_splits
            d.w = self.dense.data_ptr()
        return d

    def nbytes(self) -> int:
        return self.packed.nbytes() if self.packed is not None else self.dense.numel() * 2


def _to_device_linear(lins: Sequence, device, rows_hint: int) -> DeviceLinear:
    if all(isinstance(l, Int4Linear) for l in lins):
        lin = lins[0] if len(lins) == 1 else concat_out(list(lins))
        return DeviceLinear(packed=pack_int4(lin.to(device), device, rows_hint))
    if all(isinstance(l, DenseLinear) for l in lins):
        w = torch.cat([l.weight for l in lins], dim=0).to(device=device, dtype=torch.float16).contiguous()
        if w.shape[1] % 8:
            raise ValueError("dense projections need in_features % 8 == 0")
        return DeviceLinear(dense=w)
    raise ValueError("cannot fuse INT4 and fp16 projections into one launch")


class DeviceLayer:
    def __init__(self):
        self.type = 0
        self.in_proj = self.out_proj = self.gate_up = self.down = None
        self.ffn_norm = self.attn_norm = None
        self.q_norm = self.k_norm = None
        self.wa = self.wb = self.conv_w = self.A_log = self.dt_bias = self.la_norm = None
        self.off = (0, 0, 0, 0, -1, -1)
        self.ffn_q8 = None            # (kind, group, F, [(w, scale)] * 3) when quant_format is w8a8 / w4a8


class InferenceEngine:
    def __init__(self, config: QwenConfig, device_id: int = 0, max_seq_len: int = 2048,
                 tp_size: int = 1, tp_rank: int = 0, quant_format: str = "w4a16",
                 use_int4_attention: bool = False, engine_config: Optional[EngineConfig] = None,
                 comm=None, max_batch: int = 1):
        if not torch.cuda.is_available():
            raise RuntimeError("InferenceEngine needs a CUDA device; use models.oracle.OracleEngine on CPU")
        if quant_format not in ("w4a16", "w8a8", "w4a8"):
            raise ValueError("quant_format must be w4a16, w8a8 or w4a8")
        self.quant_format = quant_format
        self.config = config
        self.ecfg = (engine_config or EngineConfig()).replace(
            tp_size=tp_size, tp_rank=tp_rank, max_seq_len=max_seq_len, max_batch=max_batch)
        self.device = torch.device("cuda", device_id)
        torch.cuda.set_device(self.device)
        self.lib = L.lib()
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self.spec: ShardSpec = make_shard_spec(config, tp_size, tp_rank)
        self.max_seq_len, self.max_batch = max_seq_len, max_batch
        self.max_rows = L.MAX_ROWS
        self.comm = comm
        self.use_int4_attention = use_int4_attention
        self.layers: List[Optional[DeviceLayer]] = [None] * config.num_hidden_layers
        self.embed: Optional[torch.Tensor] = None
        self.lm_head: Optional[DeviceLinear] = None
        self.final_norm: Optional[torch.Tensor] = None
        self.states = SequenceStates(config, self.spec, max_seq_len, max_batch, self.device)
        self._driver = None
        self._exch_carry = 0
        self._graph_key = None
        self._tmpl_key = None
        self._ptmpl_key = None
        self._launch_counts: Dict[int, int] = {}
        self._steps = 0
        self._init_rope_tables()

    # ------------------------------------------------------------------ set-up
    @property
    def kv_cache(self):
        return self.states.kv

    @property
    def deltanet_state(self):
        return self.states.dn

    def _init_rope_tables(self):
        cfg = self.config
        half = cfg.rotary_dim // 2
        freqs = 1.0 / (cfg.rope_theta ** (torch.arange(half, dtype=torch.float64) * 2.0 / cfg.rotary_dim))
        ang = torch.arange(self.max_seq_len, dtype=torch.float64)[:, None] * freqs[None, :]
        self.cos_tab = torch.cos(ang).float().to(self.device).contiguous()
        self.sin_tab = torch.sin(ang).float().to(self.device).contiguous()

    def _h16(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=torch.float16).contiguous()

    def load_layer_weights(self, layer_idx: int, lw: Union[LayerWeights, dict]):
        """`lw` is this rank's shard in engine format (loaders and
        parallel.sharding produce it)."""
        if isinstance(lw, dict):
            lw = LayerWeights(**lw)
        cfg, dev, rh = self.config, self.device, 1
        dl = DeviceLayer()
        dl.attn_norm, dl.ffn_norm = self._h16(lw.attn_norm), self._h16(lw.ffn_norm)
        if lw.is_full:
            dl.type = 0
            dl.in_proj = _to_device_linear([lw.q, lw.q_gate, lw.k, lw.v], dev, rh)
            dl.out_proj = _to_device_linear([lw.o], dev, rh)
            dl.q_norm, dl.k_norm = self._h16(lw.q_norm), self._h16(lw.k_norm)
        else:
            dl.type = 1
            sp = self.spec
            kd = sp.n_la_k * cfg.linear_key_head_dim
            vd = sp.n_la_v * cfg.linear_value_head_dim
            parts = [lw.la_qkv, lw.la_z]
            off_a = off_b = -1
            if isinstance(lw.la_a, Int4Linear) and isinstance(lw.la_qkv, Int4Linear):
                parts += [lw.la_a, lw.la_b]
                off_a, off_b = 2 * kd + 2 * vd, 2 * kd + 2 * vd + sp.n_la_v
            elif isinstance(lw.la_a, DenseLinear) and isinstance(lw.la_qkv, DenseLinear):
                parts += [lw.la_a, lw.la_b]
                off_a, off_b = 2 * kd + 2 * vd, 2 * kd + 2 * vd + sp.n_la_v
            else:
                dl.wa, dl.wb = self._h16(lw.la_a.dense(torch.float16)), self._h16(lw.la_b.dense(torch.float16))
            dl.in_proj = _to_device_linear(parts, dev, rh)
            dl.off = (0, kd, 2 * kd, 2 * kd + vd, off_a, off_b)
            dl.out_proj = _to_device_linear([lw.la_out], dev, rh)
            dl.conv_w = self._h16(lw.la_conv1d)
            dl.A_log = lw.la_A_log.to(device=dev, dtype=torch.float32).contiguous()
            dl.dt_bias, dl.la_norm = self._h16(lw.la_dt_bias), self._h16(lw.la_norm)
        if not (isinstance(lw.gate, Int4Linear) and isinstance(lw.up, Int4Linear)):
            raise NotImplementedError("FFN projections must be INT4 (w4a16)")
        dl.gate_up = DeviceLinear(packed=pack_int4(interleave_gate_up(lw.gate.to(dev), lw.up.to(dev)), dev, rh))
        dl.down = _to_device_linear([lw.down], dev, rh)
        if self.quant_format != "w4a16":
            dl.ffn_q8 = self._convert_ffn_q8(lw.gate, lw.up, lw.down)
        self.layers[layer_idx] = dl
        self._drop_driver()

    def _convert_ffn_q8(self, gate: Int4Linear, up: Int4Linear, down: Int4Linear):
        """gate / up / down re-quantised for the INT8-activation path (reference:
        src/model/weight_loader.py:122-249): W8A8 = int8 per output channel, W4A8 = signed nibbles with the
        checkpoint's group scales.  Returns (kind, group, F, [(w, scale)] * 3) on the device."""
        from ..utils import quant as Q
        conv = Q.int4_to_w8a8 if self.quant_format == "w8a8" else Q.int4_to_w4a8
        dev = self.device
        out = []
        for lin in (gate, up, down):
            need = 64 if self.quant_format == "w8a8" else 128
            if lin.in_features % need or (self.quant_format == "w4a8" and lin.group_size % 128):
                raise ValueError(f"{self.quant_format} needs in_features % {need} == 0 (got {lin.in_features})"
                                 + (" and a group size that is a multiple of 128" if need == 128 else ""))
            w, sc = conv(lin.to(dev))
            out.append((w.contiguous(), sc.contiguous()))
        return (1 if self.quant_format == "w8a8" else 2, gate.group_size, gate.out_features, out)

    def load_final_norm(self, w: torch.Tensor):
        self.final_norm = self._h16(torch.as_tensor(w))
        self._drop_driver()

    def load_lm_head(self, w: torch.Tensor):
        """`w` is this rank's vocabulary slice [vocab_local, hidden]."""
        self.lm_head = DeviceLinear(dense=self._h16(torch.as_tensor(w)))
        self._drop_driver()

    def load_embedding(self, w: torch.Tensor):
        self.embed = self._h16(torch.as_tensor(w))
        self._drop_driver()

    def load_model(self, mw: ModelWeights):
        """`mw` must already be this rank's shard."""
        for i, lw in enumerate(mw.layers):
            self.load_layer_weights(i, lw)
        self.load_embedding(mw.embed)
        self.load_lm_head(mw.lm_head)
        self.load_final_norm(mw.final_norm)

    def init_random(self, seed: int = 0, int4_attention: bool = True, embed_std: float = 0.05):
        """Random-init weights of the benchmark's form created directly on the
        device in packed layout (no checkpoint, no host copy)."""
        cfg, sp, dev = self.config, self.spec, self.device
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed + 1000 * self.tp_rank)
        H, g = cfg.hidden_size, cfg.group_size
        ones = lambda n: torch.ones(n, dtype=torch.float16, device=dev)
        rnd = lambda K, N: DeviceLinear(packed=random_packed_int4(K, N, g, dev, gen))
        dense = lambda N, K: DeviceLinear(dense=(torch.randn(N, K, device=dev, generator=gen) * 0.02).half())
        Fp = -(-sp.ffn_local // 64) * 64
        for i in range(cfg.num_hidden_layers):
            dl = DeviceLayer()
            dl.attn_norm, dl.ffn_norm = ones(H), ones(H)
            if cfg.is_full_attention(i):
                dl.type = 0
                qd, kvd = sp.n_q * cfg.head_dim, sp.n_kv * cfg.head_dim
                dl.in_proj = rnd(H, 2 * qd + 2 * kvd) if int4_attention else dense(2 * qd + 2 * kvd, H)
                dl.out_proj = rnd(qd, H) if int4_attention else dense(H, qd)
                dl.q_norm, dl.k_norm = ones(cfg.head_dim), ones(cfg.head_dim)
            else:
                dl.type = 1
                kd = sp.n_la_k * cfg.linear_key_head_dim
                vd = sp.n_la_v * cfg.linear_value_head_dim
                dl.in_proj = rnd(H, 2 * kd + 2 * vd) if int4_attention else dense(2 * kd + 2 * vd, H)
                dl.out_proj = rnd(vd, H) if int4_attention else dense(H, vd)
                dl.off = (0, kd, 2 * kd, 2 * kd + vd, -1, -1)
                dl.wa = (torch.randn(sp.n_la_v, H, device=dev, generator=gen) * 0.02).half()
                dl.wb = (torch.randn(sp.n_la_v, H, device=dev, generator=gen) * 0.02).half()
                dl.conv_w = (torch.randn(2 * kd + vd, cfg.linear_conv_kernel_dim, device=dev, generator=gen) * 0.3).half()
                dl.A_log = (torch.rand(sp.n_la_v, device=dev, generator=gen) * 1.5 - 1.0).float()
                dl.dt_bias = (torch.randn(sp.n_la_v, device=dev, generator=gen) * 0.5).half()
                dl.la_norm = ones(cfg.linear_value_head_dim)
            dl.gate_up = rnd(H, 2 * Fp)
            if Fp != sp.ffn_local:
                raise NotImplementedError("random init needs ffn_local % 64 == 0")
            dl.down = rnd(sp.ffn_local, H)
            if self.quant_format != "w4a16":
                from ..ops.packing import unpack_fragments
                gu = unpack_fragments(dl.gate_up.packed)              # gate/up interleaved by 8
                idx = torch.arange(2 * Fp, device=dev).reshape(-1, 2, 8)
                take = lambda cols: Int4Linear(gu.qweight[:, cols].contiguous(), gu.scales[:, cols].contiguous(),
                                               None if gu.zeros is None else gu.zeros[:, cols].contiguous(), gu.group_size, 0)
                dl.ffn_q8 = self._convert_ffn_q8(take(idx[:, 0].reshape(-1)), take(idx[:, 1].reshape(-1)),
                                                 unpack_fragments(dl.down.packed))
            self.layers[i] = dl
        # replicated tensors use a rank-independent generator so every rank holds the same values
        g2 = torch.Generator(device=dev)
        g2.manual_seed(seed + 7)
        self.embed = (torch.randn(cfg.vocab_size, H, device=dev, generator=g2) * embed_std).half()
        vl = sp.vocab_local
        self.lm_head = DeviceLinear(dense=(torch.randn(vl, H, device=dev, generator=gen) * embed_std).half())
        self.final_norm = ones(H)
        self._drop_driver()

    def weight_bytes(self) -> int:
        n = sum(l.nbytes() for dl in self.layers for l in (dl.in_proj, dl.out_proj, dl.gate_up, dl.down))
        return n + self.lm_head.nbytes()

    def streamed_bytes_per_token(self) -> int:
        """Weight bytes one decode step must read (embedding row excluded)."""
        return self.weight_bytes()

    # ------------------------------------------------------------------ driver
    def _comm_ctx(self) -> L.CommCtx:
        if self.comm is not None and self.tp_size > 1:
            return self.comm.ctx()
        return L.null_comm()

    def _ensure_driver(self):
        if self._driver is not None:
            return
        if any(l is None for l in self.layers) or self.embed is None or self.lm_head is None \
                or self.final_norm is None:
            raise RuntimeError("weights are not fully loaded")
        cfg, sp, dev, R = self.config, self.spec, self.device, self.max_rows
        H = cfg.hidden_size
        lins = [l for dl in self.layers for l in (dl.in_proj, dl.out_proj, dl.gate_up, dl.down)] + [self.lm_head]
        # work buffers; with debug_guards each one sits between poisoned bands that are checked after
        # every eager step (utils/guards.py)
        self._guards = None
        if self.ecfg.debug_guards:
            from ..utils.guards import GuardedAllocator
            self._guards = GuardedAllocator(dev)
        counter = [0]

        def alloc(shape, dtype):
            if self._guards is None:
                return torch.zeros(*shape, dtype=dtype, device=dev)
            counter[0] += 1
            return self._guards.zeros(f"#{counter[0]}", shape, dtype)
        f32 = lambda *s: alloc(s, torch.float32)
        f16 = lambda *s: alloc(s, torch.float16)
        i32 = lambda *s: alloc(s, torch.int32)
        self.F_pad = self.layers[0].gate_up.n_pad // 2
        b = self.buf = {}
        b["h"], b["xn"] = f32(R, H), f16(R, H)
        # row stride of the projection buffers: widest in-projection + spare columns for the a | b gate
        # projections of many-row steps
        n_in = -(-max(dl.in_proj.N for dl in self.layers) // 8) * 8
        self.ab_off = n_in
        b["ld_proj"] = n_in + -(-max(2, 2 * sp.n_la_v) // 8) * 8
        b["proj"] = f16(R, b["ld_proj"])
        b["ld_attn"] = max(dl.out_proj.K for dl in self.layers)
        b["attn_out"] = f16(R, b["ld_attn"])
        b["act"] = f16(R, self.F_pad)
        b["ld_logits"] = -(-sp.vocab_local // 4) * 4
        b["logits"] = f32(R, b["ld_logits"])
        # split-K partial sums travel as {value, tag} pairs in the step driver: twice the floats
        self.tagged_splitk = os.environ.get("B200GRAD_TAGGED_SPLITK", "1") != "0"
        b["gemv_scratch"] = f32(2 * max(1, max(l.scratch_floats(R) for l in lins)))
        b["gemv_counters"] = i32(8192)
        # cache slices per decode-attention row: long contexts need more CTAs than (rows x KV heads) gives
        self.attn_splits = 16 if self.max_seq_len <= 1024 else 32
        G = sp.n_q // sp.n_kv
        b["attn_scratch"] = f32(R * sp.n_kv * self.attn_splits * G * (cfg.head_dim + 4))
        b["attn_counters"] = i32(R * sp.n_kv + 8)
        self.argmax_blocks = max(1, min(64, sp.vocab_local // 2048))
        b["argmax_scratch"] = f32(R * self.argmax_blocks * 2)
        b["argmax_counters"] = i32(R + 8)
        b["extra"], b["h_tmp"] = f32(R, H), f32(R, H)
        # sums of squares for the lazy RMSNorm: one entry per 64 columns (the chain kernel's tile); the
        # 128-column tiles of the stand-alone GEMV fill two entries each
        self.np = 2 * -(-H // 128)
        b["ss"] = f32(R, self.np)
        # persistent projection chain: split-K pieces and tile / dependency counters
        int4 = [l for l in lins if l.packed is not None]
        uc = int(self.ecfg.use_chain)
        self.use_chain = (2 if 1 < self.tp_size <= 4 else 0) if uc < 0 else uc
        if not int4:
            self.use_chain = 0
        self.lib.b2_chain_scratch_floats.restype = C.c_longlong
        need = max([int(self.lib.b2_chain_scratch_floats(l.packed.KB, l.packed.NTL // 4, R)) for l in int4] + [1])
        b["chain_scratch"] = f32(need)
        b["chain_counters"] = i32(8)
        # INT8-activation FFN (quant_format w8a8 / w4a8): quantised rows, their scales, gate / up / down outputs
        if any(dl.ffn_q8 is not None for dl in self.layers):
            Pq = max(R, min(512, self.max_seq_len))
            Fq = max(dl.ffn_q8[2] for dl in self.layers if dl.ffn_q8 is not None)
            b["q8_xq"] = alloc((Pq, max(H, Fq)), torch.int8)
            b["q8_sx"], b["q8_xn"] = f32(Pq), f16(Pq, H)
            b["q8_gate"], b["q8_up"], b["q8_down"] = f16(Pq, Fq), f16(Pq, Fq), f32(Pq, H)
        # tagged hand-off buffers between the projections of one chain launch ({value, tag} pairs)
        self.chain_act_cols = -(-self.F_pad // 2)
        b["chain_tag_h"], b["chain_tag_ss"] = f32(R, H, 2), f32(R, self.np, 2)
        b["chain_tag_act"] = i32(R, self.chain_act_cols, 2)
        b["rows"], b["rows_tmpl"] = i32(R, 6), i32(R, 6)
        b["row_tokens"] = torch.full((R,), -1, dtype=torch.int32, device=dev)
        b["seq_rows"] = i32(self.max_batch + 1 + R)
        b["out_tokens"] = i32(R)
        b["emb_in"] = f32(R, H)
        # prefill buffers (tensor-core path, up to max_prefill rows per launch)
        P = self.max_prefill = min(512, self.max_seq_len)
        self.use_tc_prefill = all(l.packed is not None for l in lins[:-1])
        b["p_h"], b["p_xn"] = f32(P, H), f16(P, H)
        # sequence-parallel many-row steps: the activations live in symmetric memory, where every rank's
        # reduce-scatter + norm + all-gather kernel stores its rows
        self.seq_parallel = bool(self.ecfg.seq_parallel) and self.tp_size > 1 and self.comm is not None \
            and hasattr(self.comm, "xn_view") and P * H <= getattr(self.comm, "xn_halves", 0) and H % 8 == 0 and H <= 8192
        if self.seq_parallel:
            b["p_xn"] = self.comm.xn_view(P, H)
        b["p_proj"], b["p_attn"], b["p_act"] = f16(P, b["ld_proj"]), f16(P, b["ld_attn"]), f16(P, self.F_pad)
        b["p_partial"] = f32(P, H) if self.tp_size > 1 else f32(1)
        b["p_rows"], b["p_rows_tmpl"] = i32(P, 6), i32(P, 6)
        b["p_row_tokens"] = torch.full((P,), -1, dtype=torch.int32, device=dev)
        b["tc_status"] = i32(4)
        b["p_ab"] = f16(P, max(2, 2 * sp.n_la_v))
        b["coll_counters"] = i32(8)
        # many-row steps (batched decode, speculative verification): logits / arg-max / split-KV scratch
        SR = self.step_rows = min(P, max(8, self.ecfg.max_step_rows or 8 * self.max_batch))
        b["p_logits"] = f32(SR, b["ld_logits"])
        b["p_argmax_scratch"], b["p_argmax_counters"] = f32(SR * self.argmax_blocks * 2), i32(SR + 8)
        b["p_out_tokens"] = i32(P)
        b["p_attn_scratch"] = f32(SR * sp.n_kv * self.attn_splits * G * (cfg.head_dim + 4))
        b["p_attn_counters"] = i32(SR * sp.n_kv + 8)
        # speculative verification: staging of the DeltaNet verify kernel, acceptance results
        offs = [C.c_int() for _ in range(4)]
        self.lib.b2_spec_stage_layout.restype = C.c_longlong
        blk = int(self.lib.b2_spec_stage_layout(sp.n_la_k, sp.n_la_v, cfg.linear_key_head_dim,
                                                cfg.linear_value_head_dim, *[C.byref(o) for o in offs]))
        n_lin = len(self.states.dn.layers)
        b["spec_stage"] = torch.zeros(max(1, n_lin) * self.max_batch * blk, dtype=torch.uint8, device=dev)
        b["spec_acc"] = i32(self.max_batch, L.SPEC_MAX_NODES + 2)
        b["spec_result"] = i32(self.max_batch, L.SPEC_MAX_NODES + 2)

        m = L.ModelDesc()
        m.n_layers, m.H, m.vocab = cfg.num_hidden_layers, H, cfg.vocab_size
        m.vocab_local, m.vocab_offset = sp.vocab_local, sp.vocab[0]
        m.nq, m.nkv, m.hd, m.rot = sp.n_q, sp.n_kv, cfg.head_dim, cfg.rotary_dim
        m.rope_interleaved = 1 if cfg.rope_style == "interleaved" else 0
        m.la_nk, m.la_nv = sp.n_la_k, sp.n_la_v
        m.la_dk, m.la_dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        m.max_seq, m.max_rows = self.max_seq_len, R
        m.ar_mode = AR_MODE_ID[self.ecfg.ar_mode]
        m.attn_splits, m.argmax_blocks, m.n_seqs_max = self.attn_splits, self.argmax_blocks, self.max_batch
        m.eps, m.F_pad = cfg.rms_norm_eps, self.F_pad
        m.embed, m.first_norm = self.embed.data_ptr(), self.layers[0].attn_norm.data_ptr()
        m.lm_head = self.lm_head.desc()
        m.cos_tab, m.sin_tab = self.cos_tab.data_ptr(), self.sin_tab.data_ptr()
        for k in ("h", "xn", "proj", "attn_out", "act", "logits", "gemv_scratch", "gemv_counters",
                  "attn_scratch", "attn_counters", "argmax_scratch", "argmax_counters", "extra",
                  "h_tmp", "ss", "rows", "rows_tmpl", "row_tokens", "seq_rows", "out_tokens"):
            setattr(m, k, b[k].data_ptr())
        m.ld_proj, m.ld_attn, m.ld_logits = b["ld_proj"], b["ld_attn"], b["ld_logits"]
        m.np = self.np
        m.chain_scratch, m.chain_counters = b["chain_scratch"].data_ptr(), b["chain_counters"].data_ptr()
        m.chain_act_cols, m.use_chain = self.chain_act_cols, int(self.use_chain)
        m.tagged_splitk = int(self.tagged_splitk)
        m.chain_tag_h, m.chain_tag_ss = b["chain_tag_h"].data_ptr(), b["chain_tag_ss"].data_ptr()
        m.chain_tag_act = b["chain_tag_act"].data_ptr()
        for k in ("q8_xq", "q8_sx", "q8_gate", "q8_up", "q8_down", "q8_xn"):
            if k in b:
                setattr(m, k, b[k].data_ptr())
        m.seqs = self.states.seqs.data_ptr()
        m.comm = self._comm_ctx()
        m.max_prefill = self.max_prefill
        if self.seq_parallel:
            # (a communicator rebuilt by recover() has a new symmetric block)
            b["p_xn"] = self.comm.xn_view(self.max_prefill, self.config.hidden_size)
        for k in ("p_h", "p_xn", "p_proj", "p_attn", "p_act", "p_partial", "p_rows", "p_rows_tmpl", "p_row_tokens",
                  "tc_status", "coll_counters", "p_ab"):
            setattr(m, k, b[k].data_ptr())
        for k in ("p_logits", "p_argmax_scratch", "p_argmax_counters", "p_out_tokens", "p_attn_scratch",
                  "p_attn_counters", "spec_acc", "spec_result"):
            setattr(m, k, b[k].data_ptr())
        m.p_logit_rows, m.n_lin_layers, m.n_full_layers = SR, n_lin, len(self.states.kv.layers)
        m.ab_off = self.ab_off
        m.spec.base, m.spec.layer_stride, m.spec.seq_stride = b["spec_stage"].data_ptr(), self.max_batch * blk, blk
        m.spec.off_k, m.spec.off_u, m.spec.off_g, m.spec.off_x = [o.value for o in offs]
        dn, kv = self.states.dn, self.states.kv
        if n_lin:
            m.state0, m.conv0 = dn.S.data_ptr(), dn.conv.data_ptr()
            m.state_layer_stride, m.conv_layer_stride = dn.S.stride(0), dn.conv.stride(0)
        if len(kv.layers):
            m.k0, m.v0, m.kv_layer_stride = kv.k.data_ptr(), kv.v.data_ptr(), kv.k.stride(0)
        if self.comm is not None and self.tp_size > 1:
            if self.comm.part_floats < self.max_prefill * H:
                raise ValueError("communicator staging buffer is smaller than max_prefill x hidden")
            for r in range(self.tp_size):
                m.coll_gather[r] = self.comm.peer_ptrs[r] + self.comm.off_gather
            m.coll_mc_gather = (self.comm.multicast_ptr + self.comm.off_gather) if self.comm.multicast_ptr else None
            if self.seq_parallel:
                for r in range(self.tp_size):
                    m.xn_sym[r] = self.comm.peer_ptrs[r] + self.comm.off_xn
                    m.hlast_sym[r] = self.comm.peer_ptrs[r] + self.comm.off_hlast
                m.xn_mc = (self.comm.multicast_ptr + self.comm.off_xn) if self.comm.multicast_ptr else None
                m.seq_parallel = 1
        descs = (L.LayerDesc * cfg.num_hidden_layers)()
        for i, dl in enumerate(self.layers):
            d = descs[i]
            d.type = dl.type
            d.type_index = self.states.kv.index[i] if dl.type == 0 else self.states.dn.index[i]
            d.in_proj, d.out_proj = dl.in_proj.desc(), dl.out_proj.desc()
            d.gate_up, d.down = dl.gate_up.desc(), dl.down.desc()
            d.attn_norm = dl.attn_norm.data_ptr()
            d.ffn_norm = dl.ffn_norm.data_ptr()
            nxt = self.layers[i + 1].attn_norm if i + 1 < len(self.layers) else self.final_norm
            d.next_norm = nxt.data_ptr()
            if dl.type == 0:
                d.q_norm, d.k_norm = dl.q_norm.data_ptr(), dl.k_norm.data_ptr()
                d.kcache = self.states.kv.layer_k(i).data_ptr()
                d.vcache = self.states.kv.layer_v(i).data_ptr()
            else:
                d.wa = None if dl.wa is None else dl.wa.data_ptr()
                d.wb = None if dl.wb is None else dl.wb.data_ptr()
                if dl.wa is not None and dl.wb is not None:
                    if getattr(dl, "wab", None) is None:
                        dl.wab = torch.cat([dl.wa, dl.wb], dim=0).contiguous()
                    d.wab = dl.wab.data_ptr()
                d.conv_w, d.A_log = dl.conv_w.data_ptr(), dl.A_log.data_ptr()
                d.dt_bias, d.la_norm = dl.dt_bias.data_ptr(), dl.la_norm.data_ptr()
                d.conv_state = self.states.dn.layer_conv(i).data_ptr()
                d.state = self.states.dn.layer_S(i).data_ptr()
                d.off_q, d.off_k, d.off_v, d.off_z, d.off_a, d.off_b = dl.off
            if dl.ffn_q8 is not None:
                d.ffn_kind, d.q8_group, d.q8_F, ws = dl.ffn_q8
                for j, (w, sc) in enumerate(ws):
                    d.q8_w[j], d.q8_s[j] = w.data_ptr(), sc.data_ptr()
        self._model_desc, self._layer_descs = m, descs
        self._driver = self.lib.b2_driver_create(C.byref(m), descs)
        self._graph_key = None
        self._tmpl_key = None
        self._stream = torch.cuda.Stream(device=dev)

    def build_decode_launch_cache(self):
        """Reference-compatible name (src/inference/engine.py:3309): builds the
        driver plan."""
        self._ensure_driver()

    # ------------------------------------------------------------------ rows
    def _set_template(self, key, rows: List[tuple], seq_rows: List[int]):
        """rows: (seq, depth, slot_offset, mask) per row."""
        if key is not None and key == self._tmpl_key:
            return
        t = torch.zeros(self.max_rows, 6, dtype=torch.int32)
        for r, (seq, depth, slot, mask) in enumerate(rows):
            t[r, 0], t[r, 1], t[r, 2] = seq, depth, slot
            t[r, 4] = (mask & 0xFFFFFFFF) - (1 << 32 if mask & 0x80000000 else 0)
            hi = (mask >> 32) & 0xFFFFFFFF
            t[r, 5] = hi - (1 << 32 if hi & 0x80000000 else 0)
        self.buf["rows_tmpl"].copy_(t.to(self.device))
        sr = torch.zeros(self.buf["seq_rows"].shape[0], dtype=torch.int32)
        sr[:len(seq_rows)] = torch.tensor(seq_rows, dtype=torch.int32)
        self.buf["seq_rows"].copy_(sr.to(self.device))
        self._tmpl_key = key

    def _template_decode(self, seqs: Sequence[int]):
        self._set_template(("decode", tuple(seqs)), [(s, 0, 0, 1) for s in seqs],
                           list(range(len(seqs) + 1)))

    def _template_chain(self, seq: int, n: int):
        self._set_template(("chain", seq, n), [(seq, i, i, (1 << (i + 1)) - 1) for i in range(n)], [0, n])

    def _run(self, rows: int, n_seqs: int, flags: int):
        self._ensure_driver()
        L.check(self.lib.b2_driver_step(C.c_void_p(self._driver), rows, n_seqs, flags, L.stream()), "driver step")
        self._steps += 1
        if self._guards is not None:
            self.check_guards()

    def check_guards(self):
        """debug_guards: synchronise and verify that no kernel wrote outside a work buffer; the
        report names buffers by their key in `self.buf`."""
        if self._guards is None:
            return
        torch.cuda.synchronize(self.device)
        from ..utils.guards import GuardError
        try:
            self._guards.check_all()
        except GuardError as e:
            names = {t.data_ptr(): k for k, t in self.buf.items() if torch.is_tensor(t)}
            by_ptr = {raw[self._guards.band:].data_ptr(): n for n, (raw, _) in self._guards._bufs.items()}
            alias = {n: names.get(p, n) for p, n in by_ptr.items()}
            msg = str(e)
            for n, k in alias.items():
                msg = msg.replace(f"{n}:", f"{k}:")
            raise GuardError(msg) from None

    # ------------------------------------------------------------------ token-level API
    def step_tokens(self, tokens: Sequence[int], seq: int = 0, logits: bool = True,
                    commit: bool = True) -> torch.Tensor:
        """Feed `tokens` (<= 8) of one sequence as a chain; returns the arg-max
        token after every fed token (device int32 [n])."""
        n = len(tokens)
        if not 1 <= n <= self.max_rows:
            raise ValueError(f"1..{self.max_rows} tokens per step")
        self._ensure_driver()
        self._template_chain(seq, n)
        rt = torch.full((self.max_rows,), -1, dtype=torch.int32)
        rt[:n] = torch.as_tensor(list(tokens), dtype=torch.int32)
        self.buf["row_tokens"].copy_(rt.to(self.device))
        flags = L.STEP_EMBED_TOKENS | ((L.STEP_LM_HEAD | L.STEP_ARGMAX) if logits else 0)
        if not commit:
            flags |= L.STEP_NO_COMMIT_DELTA
        self._run(n, 1, flags)
        if commit:
            self.states.seqs[seq, 0] += n
        self.buf["row_tokens"].fill_(-1)
        return self.buf["out_tokens"][:n]

    def _prefill_rows(self, n: int, seq: int, flags: int):
        """Run n rows (already staged: tokens in p_row_tokens or embeddings in p_h/p_xn) of one
        sequence through the tensor-core prefill path and commit them."""
        t = torch.zeros(n, 6, dtype=torch.int32)
        idx = torch.arange(n, dtype=torch.int32)
        t[:, 0], t[:, 1], t[:, 2], t[:, 3] = seq, idx, idx, idx + 1      # pos, slot, visible new slots
        self.buf["p_rows_tmpl"][:n].copy_(t.to(self.device))
        sr = torch.zeros(self.buf["seq_rows"].shape[0], dtype=torch.int32)
        sr[1] = n
        self.buf["seq_rows"].copy_(sr.to(self.device))
        self._tmpl_key = self._ptmpl_key = None
        L.check(self.lib.b2_driver_prefill(C.c_void_p(self._driver), n, flags, L.stream()), "driver prefill")
        self.states.seqs[seq, 0] += n
        self._steps += 1

    def prefill_tokens_tc(self, tokens: Sequence[int], seq: int = 0) -> int:
        """Prompt processing on the tcgen05 GEMM path, max_prefill rows per launch; returns the
        first generated token."""
        self._ensure_driver()
        from ..ops import kernels as K
        tokens = list(tokens)
        n = 0
        for i in range(0, len(tokens), self.max_prefill):
            chunk = tokens[i:i + self.max_prefill]
            n = len(chunk)
            self.buf["p_row_tokens"][:n].copy_(torch.tensor(chunk, dtype=torch.int32).to(self.device))
            self._prefill_rows(n, seq, L.STEP_EMBED_TOKENS)
        # logits of the last row: final-normed hidden state is in p_xn[n-1]
        K.gemv(self.lm_head, self.buf["p_xn"][n - 1:n], out=self.buf["logits"][:1], mode=L.EPI_STORE_F32,
               scratch=self.buf["gemv_scratch"], counters=self.buf["gemv_counters"])
        tok = K.argmax(self.buf["logits"][:1, :self.spec.vocab_local], self.spec.vocab[0], self.argmax_blocks,
                       self._comm_ctx() if self.tp_size > 1 else None)
        self.buf["h"][:1].copy_(self.buf["p_h"][n - 1:n])
        self.states.seqs[seq, 1] = tok[0]
        return int(tok[0].item())

    def score_tokens(self, tokens: Sequence[int], seq: int = 0) -> torch.Tensor:
        """Teacher-forced log-probabilities: feeds `tokens` to an empty sequence slot and returns
        log p(tokens[i+1] | tokens[:i+1]) for i = 0 .. n-2 (fp32, device).  Rows go through the
        many-row path in launches of `step_rows`, with the lm_head applied to every row.  Under
        tensor parallelism the vocabulary slices are combined with two small all-reduces."""
        self._ensure_driver()
        if not self.use_tc_prefill:
            raise NotImplementedError("scoring uses the tensor-core path (all projections INT4)")
        tokens = [int(t) for t in tokens]
        self.states.reset(seq)
        out = []
        a, b = self.spec.vocab
        for i in range(0, len(tokens), self.step_rows):
            chunk = tokens[i:i + self.step_rows]
            n = len(chunk)
            self.buf["p_row_tokens"][:n].copy_(torch.tensor(chunk, dtype=torch.int32).to(self.device))
            self._prefill_rows(n, seq, L.STEP_EMBED_TOKENS | L.STEP_LM_HEAD)
            nxt = torch.tensor(tokens[i + 1:i + 1 + n], dtype=torch.long, device=self.device)
            m = nxt.numel()
            if m == 0:
                break
            lg = self.buf["p_logits"][:m, :self.spec.vocab_local]
            mx = lg.max(dim=-1).values
            local = (nxt >= a) & (nxt < b)
            tgt = torch.where(local, lg.gather(1, (nxt - a).clamp(0, self.spec.vocab_local - 1)[:, None])[:, 0],
                              torch.zeros_like(mx))
            if self.tp_size > 1:
                import torch.distributed as dist
                dist.all_reduce(mx, op=dist.ReduceOp.MAX)
                dist.all_reduce(tgt)
            se = torch.exp(lg - mx[:, None]).sum(dim=-1)
            if self.tp_size > 1:
                import torch.distributed as dist
                dist.all_reduce(se)
            out.append(tgt - mx - torch.log(se))
        return torch.cat(out) if out else torch.zeros(0, device=self.device)

    def perplexity(self, tokens: Sequence[int], seq: int = 0) -> float:
        lp = self.score_tokens(tokens, seq)
        return float(torch.exp(-lp.mean()).item()) if lp.numel() else float("nan")

    def prefill_tokens(self, tokens: Sequence[int], seq: int = 0) -> int:
        """Consume a prompt; returns the first generated token and stores it as
        the sequence's next input."""
        tokens = list(tokens)
        self._ensure_driver()
        if self.use_tc_prefill and len(tokens) >= 16:
            return self.prefill_tokens_tc(tokens, seq)
        out = None
        for i in range(0, len(tokens), self.max_rows):
            chunk = tokens[i:i + self.max_rows]
            last = i + self.max_rows >= len(tokens)
            out = self.step_tokens(chunk, seq, logits=last)
        n = len(chunk)
        tok = out[n - 1]
        if n > 1:
            # the prompt's last row becomes row 0, where logits() and compute_logits(None) look
            self.buf["logits"][0].copy_(self.buf["logits"][n - 1])
            self.buf["h"][0].copy_(self.buf["h"][n - 1])
        self.states.seqs[seq, 1] = tok
        return int(tok.item())

    def decode_tokens(self, n_steps: int, seqs: Optional[Sequence[int]] = None, graph: Optional[bool] = None,
                      collect: bool = True) -> Optional[torch.Tensor]:
        """Greedy-decode `n_steps` tokens for the given sequence slots; each step
        consumes SeqState.token and writes the next one.  Returns int32
        [n_steps, len(seqs)] when `collect`."""
        seqs = list(seqs) if seqs is not None else [0]
        self._ensure_driver()
        rows = len(seqs)
        flags = L.STEP_EMBED_TOKENS | L.STEP_LM_HEAD | L.STEP_ARGMAX | L.STEP_ADVANCE
        out_buf = self.buf["out_tokens"]
        if rows > self.max_rows:
            # more sequences than the GEMV kernels take rows: tensor-core path
            if not self.use_tc_prefill or rows > self.step_rows:
                raise ValueError(f"{rows} sequences exceed what this engine was sized for ({self.step_rows})")
            key = ("decode", tuple(seqs))
            if self._ptmpl_key != key:
                t = torch.zeros(rows, 6, dtype=torch.int32)
                t[:, 0] = torch.tensor(seqs, dtype=torch.int32)
                t[:, 4] = 1
                self.buf["p_rows_tmpl"][:rows].copy_(t.to(self.device))
                sr = torch.zeros(self.buf["seq_rows"].shape[0], dtype=torch.int32)
                sr[:rows + 1] = torch.arange(rows + 1, dtype=torch.int32)
                self.buf["seq_rows"].copy_(sr.to(self.device))
                self.buf["p_row_tokens"][:rows].fill_(-1)
                self._ptmpl_key, self._tmpl_key = key, None
            flags |= L.STEP_GEMM_PATH
            out_buf = self.buf["p_out_tokens"]
        else:
            self._template_decode(seqs)
        use_graph = self.ecfg.use_graph if graph is None else graph
        outs = []
        if use_graph:
            key = ("decode", tuple(seqs), flags)
            if self._graph_key != key:
                torch.cuda.synchronize()
                with torch.cuda.stream(self._stream):
                    L.check(self.lib.b2_driver_capture(C.c_void_p(self._driver), rows, rows, flags,
                                                       C.c_void_p(self._stream.cuda_stream)), "graph capture")
                torch.cuda.synchronize()
                self._graph_key = key
            if collect:
                for _ in range(n_steps):
                    L.check(self.lib.b2_driver_replay(C.c_void_p(self._driver), 1, L.stream()), "graph replay")
                    outs.append(out_buf[:rows].clone())
            else:
                L.check(self.lib.b2_driver_replay(C.c_void_p(self._driver), n_steps, L.stream()), "graph replay")
        else:
            for _ in range(n_steps):
                self._run(rows, rows, flags)
                if collect:
                    outs.append(out_buf[:rows].clone())
        self._steps += n_steps
        return torch.stack(outs) if collect else None

    def generate_tokens(self, prompt: Sequence[int], n_new: int, seq: int = 0, graph: Optional[bool] = None):
        """Greedy generation entirely on the device: returns n_new token ids."""
        self.states.reset(seq)
        first = self.prefill_tokens(prompt, seq)
        if n_new <= 1:
            return [first][:n_new]
        rest = self.decode_tokens(n_new - 1, [seq], graph=graph)
        return [first] + rest[:, 0].tolist()

    def step_host(self, token: int, seq: int = 0) -> int:
        """One greedy decode step driven from the host: the input token is
        uploaded from pinned memory, the step graph is replayed, the next token is
        downloaded.  This is the per-token path of the generation API."""
        self._ensure_driver()
        if not hasattr(self, "_pin_in"):
            self._pin_in = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._pin_out = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._pin_in[0] = int(token)
        self.states.seqs[seq, 1:2].copy_(self._pin_in, non_blocking=True)
        self.decode_tokens(1, [seq], collect=False)
        self._pin_out.copy_(self.buf["out_tokens"][:1], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return int(self._pin_out[0])

    # ------------------------------------------------------------------ speculative verification
    def spec_step(self, drafts: Sequence[Sequence[int]], parents: Sequence[Sequence[int]],
                  seqs: Optional[Sequence[int]] = None, roots: Optional[Sequence[int]] = None,
                  graph: bool = False, tokens_dev: Optional[torch.Tensor] = None, sync: bool = True):
        """One verify-and-commit step for several sequences.  For sequence i the
        pending token (roots[i], default: the token the last step stored) and the
        draft tree drafts[i] / parents[i] (parent -1 = child of the pending token,
        parents precede children) go through the model in ONE pass; the longest
        path the model would have produced greedily is accepted on the device and
        KV cache, DeltaNet state and sequence length end up as if only the accepted
        tokens had been fed.  Returns [(accepted draft tokens, next pending token)].

        `graph`: replay the step from a CUDA graph captured for this tree shape.
        `tokens_dev`: int32 device tensor with the row tokens (pending token or -1,
        then the drafts, per sequence) instead of the host lists in `drafts`, whose
        values are then ignored.  `sync=False` skips the result download (read
        `buf["spec_result"]` later)."""
        seqs = list(seqs) if seqs is not None else list(range(len(drafts)))
        self._ensure_driver()
        n_seqs = len(seqs)
        if n_seqs > self.max_batch or len(drafts) != n_seqs or len(parents) != n_seqs:
            raise ValueError("one draft list per sequence, at most max_batch sequences")
        rows, seq_rows, toks = [], [0], []
        for i, sq in enumerate(seqs):
            d, par = list(drafts[i]), list(parents[i])
            if len(d) != len(par) or len(d) + 1 > L.SPEC_MAX_NODES:
                raise ValueError(f"a draft tree has at most {L.SPEC_MAX_NODES - 1} nodes")
            masks, depth = [1], [0]
            for t, pp in enumerate(par):
                if not -1 <= pp < t:
                    raise ValueError("parents must precede their children")
                masks.append(masks[pp + 1] | (1 << (t + 1)))
                depth.append(depth[pp + 1] + 1)
            for t in range(len(d) + 1):
                rows.append((sq, depth[t], t, masks[t]))
            toks += [-1 if roots is None else int(roots[i])] + [int(x) for x in d]
            seq_rows.append(len(rows))
        R = len(rows)
        gemm_path = R > self.max_rows
        if gemm_path and (not self.use_tc_prefill or R > self.step_rows):
            raise ValueError(f"{R} rows exceed what this engine was sized for ({self.step_rows})")
        key = ("spec", tuple(rows))
        flags = L.STEP_EMBED_TOKENS | L.STEP_LM_HEAD | L.STEP_ARGMAX | L.STEP_SPEC
        if gemm_path:
            flags |= L.STEP_GEMM_PATH
            if self._ptmpl_key != key:
                t = torch.zeros(R, 6, dtype=torch.int32)
                for r, (sq, dep, slot, mask) in enumerate(rows):
                    t[r, 0], t[r, 1], t[r, 2], t[r, 4] = sq, dep, slot, mask
                self.buf["p_rows_tmpl"][:R].copy_(t.to(self.device))
                sr = torch.zeros(self.buf["seq_rows"].shape[0], dtype=torch.int32)
                sr[:len(seq_rows)] = torch.tensor(seq_rows, dtype=torch.int32)
                self.buf["seq_rows"].copy_(sr.to(self.device))
                self._ptmpl_key, self._tmpl_key = key, None
            tok_buf = self.buf["p_row_tokens"]
        else:
            self._set_template(key, rows, seq_rows)
            self._ptmpl_key = None
            tok_buf = self.buf["row_tokens"]
        if tokens_dev is not None:
            tok_buf[:R].copy_(tokens_dev[:R], non_blocking=True)
        else:
            tok_buf[:R].copy_(torch.tensor(toks, dtype=torch.int32).to(self.device))
        if graph:
            gkey = ("spec", key, flags)
            if self._graph_key != gkey:
                torch.cuda.synchronize()
                with torch.cuda.stream(self._stream):
                    L.check(self.lib.b2_driver_capture(C.c_void_p(self._driver), R, n_seqs, flags,
                                                       C.c_void_p(self._stream.cuda_stream)), "graph capture")
                torch.cuda.synchronize()
                self._graph_key = gkey
            L.check(self.lib.b2_driver_replay(C.c_void_p(self._driver), 1, L.stream()), "graph replay")
            self._steps += 1
        else:
            self._run(R, n_seqs, flags)
        if not gemm_path:
            self.buf["row_tokens"].fill_(-1)
        if not sync:
            return None
        res = self.buf["spec_result"][:n_seqs].tolist()
        return [(r[2:2 + r[0]], r[1]) for r in res]

    def spec_step_tokens(self, root: int, drafts: Sequence[int], parents: Sequence[int], seq: int = 0):
        """Single-sequence form used by generate.speculative.EngineBackend."""
        return self.spec_step([list(drafts)], [list(parents)], [seq], [root])[0]

    def logits(self, rows: int = 1) -> torch.Tensor:
        """fp32 logits of the last step, this rank's vocabulary slice."""
        return self.buf["logits"][:rows, :self.spec.vocab_local]

    # ------------------------------------------------------------------ embedding-in API
    def _as_dev(self, x) -> torch.Tensor:
        if isinstance(x, np.ndarray):
            x = torch.from_numpy(x)
        return x.to(device=self.device, dtype=torch.float32)

    def forward_embeddings(self, embs, seq: int = 0, commit: bool = True) -> torch.Tensor:
        """Run n <= 8 rows given as embeddings; returns the final-normed hidden
        states fp16 [n, hidden] (device)."""
        self._ensure_driver()
        e = self._as_dev(embs).reshape(-1, self.config.hidden_size)
        n = e.shape[0]
        self._template_chain(seq, n)
        self.buf["emb_in"][:n].copy_(e)
        L.check(self.lib.b2_load_rmsnorm(None, C.c_void_p(self.buf["emb_in"].data_ptr()),
                                         C.c_void_p(self.layers[0].attn_norm.data_ptr()),
                                         C.c_void_p(self.buf["h"].data_ptr()), None,
                                         C.c_void_p(self.buf["ss"].data_ptr()), self.np, n,
                                         self.config.hidden_size, C.c_float(self.config.rms_norm_eps),
                                         L.stream()), "load_rmsnorm")
        self._run(n, 1, L.STEP_MATERIALIZE_XN | (0 if commit else L.STEP_NO_COMMIT_DELTA))
        if commit:
            self.states.seqs[seq, 0] += n
        return self.buf["xn"][:n]

    def forward_embeddings_tree(self, embs, parents: Sequence[int], seq: int = 0) -> torch.Tensor:
        """Verify-only pass over a draft tree given as embeddings (<= 8 nodes; node 0
        is the root with parent -1, parents precede children): returns the
        final-normed hidden state of every node; KV slots beyond the committed
        length are scratch and the DeltaNet state is untouched."""
        self._ensure_driver()
        e = self._as_dev(embs).reshape(-1, self.config.hidden_size)
        n = e.shape[0]
        if n > self.max_rows or len(parents) != n or parents[0] != -1:
            raise ValueError(f"1..{self.max_rows} nodes, parents[0] == -1")
        masks, depth = [], []
        for t, pp in enumerate(parents):
            if t and not 0 <= pp < t:
                raise ValueError("parents must precede their children")
            masks.append((masks[pp] if t else 0) | (1 << t))
            depth.append(depth[pp] + 1 if t else 0)
        self._set_template(("tree", seq, tuple(parents)), [(seq, depth[t], t, masks[t]) for t in range(n)], [0, n])
        self.buf["emb_in"][:n].copy_(e)
        L.check(self.lib.b2_load_rmsnorm(None, C.c_void_p(self.buf["emb_in"].data_ptr()),
                                         C.c_void_p(self.layers[0].attn_norm.data_ptr()),
                                         C.c_void_p(self.buf["h"].data_ptr()), None,
                                         C.c_void_p(self.buf["ss"].data_ptr()), self.np, n,
                                         self.config.hidden_size, C.c_float(self.config.rms_norm_eps),
                                         L.stream()), "load_rmsnorm")
        self._run(n, 1, L.STEP_MATERIALIZE_XN | L.STEP_SPEC)
        return self.buf["xn"][:n]

    def decode_step(self, token_embedding, position: Optional[int] = None, seq: int = 0):
        """Reference signature (src/inference/engine.py:1417): embedding [hidden]
        in, final-normed hidden state out (numpy fp16 if numpy came in)."""
        if position is not None and position != self.states.length(seq):
            self.states.set_length(seq, position)
        out = self.forward_embeddings(token_embedding, seq)[0]
        return out.cpu().numpy() if isinstance(token_embedding, np.ndarray) else out.clone()

    def prefill_step(self, token_embeddings, seq: int = 0):
        """Whole prompt [S, hidden] in, hidden state of the last token out
        (reference: src/inference/engine.py:3009-3294)."""
        e = self._as_dev(token_embeddings).reshape(-1, self.config.hidden_size).contiguous()
        self._ensure_driver()
        if self.use_tc_prefill and e.shape[0] >= 16:
            # many rows: the tensor-core prefill path, max_prefill rows per launch, embeddings loaded
            # straight into its residual stream (a 512-row prompt is one launch sequence, not 64 decode steps)
            H, n = self.config.hidden_size, 0
            for i in range(0, e.shape[0], self.max_prefill):
                chunk = e[i:i + self.max_prefill]
                n = chunk.shape[0]
                L.check(self.lib.b2_load_rmsnorm(None, C.c_void_p(chunk.data_ptr()),
                                                 C.c_void_p(self.layers[0].attn_norm.data_ptr()),
                                                 C.c_void_p(self.buf["p_h"].data_ptr()),
                                                 C.c_void_p(self.buf["p_xn"].data_ptr()), None, 0, n, H,
                                                 C.c_float(self.config.rms_norm_eps), L.stream()), "load_rmsnorm")
                self._prefill_rows(n, seq, 0)
            self.buf["h"][:1].copy_(self.buf["p_h"][n - 1:n])
            out = self.buf["p_xn"][n - 1]
        else:
            out = None
            for i in range(0, e.shape[0], self.max_rows):
                out = self.forward_embeddings(e[i:i + self.max_rows], seq)
            out = out[-1]
        return out.cpu().numpy() if isinstance(token_embeddings, np.ndarray) else out.clone()

    def decode_step_batch(self, token_embeddings, batch_size: Optional[int] = None, position: Optional[int] = None,
                          seq: int = 0):
        """Several tokens of one sequence at consecutive positions in one step, embeddings in,
        final-normed hidden states out (reference: src/inference/engine.py:1513-1759, whose
        DeltaNet branch of this call fabricates outputs).  Independent sequences are decoded
        together with `decode_tokens(seqs=[...])`."""
        e = self._as_dev(token_embeddings).reshape(-1, self.config.hidden_size)
        if batch_size is not None:
            e = e[:batch_size]
        if position is not None and position != self.states.length(seq):
            self.states.set_length(seq, position)
        out = self.forward_embeddings(e, seq)
        return out.cpu().numpy() if isinstance(token_embeddings, np.ndarray) else out.clone()

    def register_tp_peers(self, *args, **kwargs):
        """The reference hands every engine its peers' buffer pointers for in-kernel peer reads
        (src/inference/engine.py, register_tp_peers).  Here peers are reached through the
        communicator's symmetric memory, which is set up at construction: nothing to register."""

    def residual_stream(self, rows: int = 1) -> torch.Tensor:
        """fp32 residual stream after the last step (before the final norm)."""
        return self.buf["h"][:rows]

    def compute_logits(self, hidden=None) -> torch.Tensor:
        """Logits (fp32, this rank's vocabulary slice) of a final-normed hidden
        state; None = the last step's (reference: src/inference/engine.py:1123-1143)."""
        self._ensure_driver()
        from ..ops import kernels as K
        if hidden is not None:
            hdn = self._as_dev(hidden).reshape(1, -1)
            self.buf["xn"][:1].copy_(hdn.half())
            x, ln = self.buf["xn"][:1], None
        else:
            # the norm is taken from the hidden state itself: the running sum of squares that the
            # step's kernels hand to one another is not kept for rows moved by a prefill
            x, ln = K.add_rmsnorm(self.buf["h"][:1], self.final_norm, eps=self.config.rms_norm_eps), None
        K.gemv(self.lm_head, x, out=self.buf["logits"][:1], mode=L.EPI_STORE_F32, ln=ln, rows=1,
               scratch=self.buf["gemv_scratch"], counters=self.buf["gemv_counters"])
        out = self.buf["logits"][0, :self.spec.vocab_local]
        return out.cpu().numpy() if isinstance(hidden, np.ndarray) else out.clone()

    # ------------------------------------------------------------------ misc reference-compatible
    def set_awq_mode(self, enabled: bool = True):
        """AWQ weights are the same packed layout with zero = 0; nothing to switch."""

    def set_direct_kv_write(self, enabled: bool = True):
        """K/V are always written straight into the cache by qknorm_rope_cachew."""

    def reset_launch_counters(self):
        self._launch_counts.clear()

    def get_layer_launch_count(self, layer_idx: int) -> int:
        """Kernels the driver issued inside this layer's part of the most recent step (issued or
        captured); 0 before the first step (reference: src/inference/engine.py:993-1023).  A chain
        launch that spans two layers counts for the layer in which it is issued."""
        self._ensure_driver()
        return max(0, int(self.lib.b2_driver_layer_launches(C.c_void_p(self._driver), layer_idx)))

    def _drop_driver(self):
        """Forget the driver plan (weights or settings changed); the counters it kept are carried over."""
        if getattr(self, "_driver", None) is not None:
            self._exch_carry += int(self.lib.b2_driver_total_exchanges(C.c_void_p(self._driver)))
            self.lib.b2_driver_destroy(C.c_void_p(self._driver))
        self._driver = None

    def exchange_count(self) -> int:
        """Cross-GPU exchanges (all-reduces fused into kernels) since the driver was built, counted
        by the driver as it issues or replays steps."""
        if self._driver is None:
            return self._exch_carry
        return self._exch_carry + int(self.lib.b2_driver_total_exchanges(C.c_void_p(self._driver)))

    def launches_per_step(self) -> int:
        self._ensure_driver()
        return int(self.lib.b2_driver_launches(C.c_void_p(self._driver)))

    def synchronize(self):
        torch.cuda.synchronize(self.device)

    def reset(self, seq: Optional[int] = None):
        self.states.reset(seq)

    def check_status(self):
        if self.comm is not None:
            self.comm.check_status()

    def cleanup(self):
        self._drop_driver()
        self.buf = {}
