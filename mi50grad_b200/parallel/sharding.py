"""Tensor-parallel weight sharder.

Column-parallel (split of the output features, by heads) for q, q_gate, k, v,
the DeltaNet in-projections and the FFN gate/up; row-parallel (split of the
input features) for o_proj, the DeltaNet out_proj and the FFN down projection
(reference: src/inference/engine.py:1145-1270).  Norms, embeddings and the final
norm are replicated; the lm_head is vocabulary-sharded so every rank computes
1/tp of the logits (the reference computes all logits on GPU 0:
src/inference/tp_engine.py:2529-2530).

Two things the reference cannot do are handled here:
* tp_size > num_key_value_heads: each KV head is replicated on tp/kv ranks
  (the reference computes 4 // 8 = 0 local KV heads: src/inference/engine.py:498);
* row shards that begin or end inside a quantisation group: the shard keeps
  every group it touches and records `group_offset`.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import List, Sequence, Tuple

import torch

from ..config import QwenConfig
from ..models.weights import LayerWeights, Linear, ModelWeights
from ..utils.quant import DenseLinear, Int4Linear, NIBBLES


@dataclass(frozen=True)
class ShardSpec:
    tp_size: int
    tp_rank: int
    q_heads: Tuple[int, int]       # [begin, end) global query-head range
    kv_heads: Tuple[int, int]      # [begin, end) global KV-head range held here
    kv_replication: int            # ranks holding the same KV head
    la_k_heads: Tuple[int, int]
    la_v_heads: Tuple[int, int]
    ffn: Tuple[int, int]           # [begin, end) of the intermediate dimension
    vocab: Tuple[int, int]

    @property
    def n_q(self) -> int:
        return self.q_heads[1] - self.q_heads[0]

    @property
    def n_kv(self) -> int:
        return self.kv_heads[1] - self.kv_heads[0]

    @property
    def n_la_k(self) -> int:
        return self.la_k_heads[1] - self.la_k_heads[0]

    @property
    def n_la_v(self) -> int:
        return self.la_v_heads[1] - self.la_v_heads[0]

    @property
    def ffn_local(self) -> int:
        return self.ffn[1] - self.ffn[0]

    @property
    def vocab_local(self) -> int:
        return self.vocab[1] - self.vocab[0]


def _even(total: int, tp: int, rank: int, what: str, multiple: int = 1) -> Tuple[int, int]:
    if total % (tp * multiple):
        raise ValueError(f"{what}={total} is not divisible by tp_size*{multiple}={tp * multiple}")
    per = total // tp
    return rank * per, (rank + 1) * per


def make_shard_spec(cfg: QwenConfig, tp_size: int, tp_rank: int) -> ShardSpec:
    if not 0 <= tp_rank < tp_size:
        raise ValueError("tp_rank out of range")
    q = _even(cfg.num_attention_heads, tp_size, tp_rank, "num_attention_heads")
    nkv = cfg.num_key_value_heads
    group = cfg.num_attention_heads // nkv
    if tp_size <= nkv:
        kv = _even(nkv, tp_size, tp_rank, "num_key_value_heads")
        rep = 1
    else:
        if tp_size % nkv:
            raise ValueError("tp_size must be a multiple of num_key_value_heads when larger")
        rep = tp_size // nkv
        kv0 = q[0] // group
        if (q[1] - 1) // group != kv0:
            raise ValueError("local query heads straddle KV heads")
        kv = (kv0, kv0 + 1)
    vocab_per = -(-cfg.vocab_size // tp_size)
    vocab = (min(cfg.vocab_size, tp_rank * vocab_per), min(cfg.vocab_size, (tp_rank + 1) * vocab_per))
    return ShardSpec(
        tp_size, tp_rank, q, kv, rep,
        _even(cfg.linear_num_key_heads, tp_size, tp_rank, "linear_num_key_heads"),
        _even(cfg.linear_num_value_heads, tp_size, tp_rank, "linear_num_value_heads"),
        _even(cfg.intermediate_size, tp_size, tp_rank, "intermediate_size", NIBBLES),
        vocab)


# -- slicing primitives -----------------------------------------------------

def slice_out(lin: Linear, ranges: Sequence[Tuple[int, int]]) -> Linear:
    """Keep the output features in `ranges` (concatenated in order)."""
    idx = torch.cat([torch.arange(a, b) for a, b in ranges])
    if isinstance(lin, DenseLinear):
        return DenseLinear(lin.weight[idx.to(lin.weight.device)].contiguous())
    idx = idx.to(lin.qweight.device)
    return Int4Linear(lin.qweight[:, idx].contiguous(), lin.scales[:, idx].contiguous(),
                      None if lin.zeros is None else lin.zeros[:, idx].contiguous(),
                      lin.group_size, lin.group_offset)


def slice_in(lin: Linear, k0: int, k1: int) -> Linear:
    """Keep input features [k0, k1)."""
    if isinstance(lin, DenseLinear):
        return DenseLinear(lin.weight[:, k0:k1].contiguous())
    if k0 % NIBBLES or k1 % NIBBLES:
        raise ValueError("row shards of packed INT4 weights must be multiples of 8")
    g, off = lin.group_size, lin.group_offset
    g0 = (k0 + off) // g
    g1 = -(-(k1 + off) // g)
    return Int4Linear(lin.qweight[k0 // NIBBLES:k1 // NIBBLES].contiguous(),
                      lin.scales[g0:g1].contiguous(),
                      None if lin.zeros is None else lin.zeros[g0:g1].contiguous(),
                      g, (k0 + off) % g)


def _head_rows(heads: Tuple[int, int], hd: int, base: int = 0) -> Tuple[int, int]:
    return base + heads[0] * hd, base + heads[1] * hd


def shard_layer(lw: LayerWeights, cfg: QwenConfig, tp_size: int, tp_rank: int) -> LayerWeights:
    if tp_size == 1:
        return lw
    sp = make_shard_spec(cfg, tp_size, tp_rank)
    out = dataclasses.replace(lw)
    out.gate = slice_out(lw.gate, [sp.ffn])
    out.up = slice_out(lw.up, [sp.ffn])
    out.down = slice_in(lw.down, *sp.ffn)
    if lw.is_full:
        hd = cfg.head_dim
        out.q = slice_out(lw.q, [_head_rows(sp.q_heads, hd)])
        out.q_gate = slice_out(lw.q_gate, [_head_rows(sp.q_heads, hd)])
        out.k = slice_out(lw.k, [_head_rows(sp.kv_heads, hd)])
        out.v = slice_out(lw.v, [_head_rows(sp.kv_heads, hd)])
        out.o = slice_in(lw.o, *_head_rows(sp.q_heads, hd))
    else:
        kd, vd = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        kdim = cfg.linear_attn_key_dim
        qkv_ranges = [_head_rows(sp.la_k_heads, kd, 0), _head_rows(sp.la_k_heads, kd, kdim),
                      _head_rows(sp.la_v_heads, vd, 2 * kdim)]
        out.la_qkv = slice_out(lw.la_qkv, qkv_ranges)
        out.la_z = slice_out(lw.la_z, [_head_rows(sp.la_v_heads, vd)])
        out.la_a = slice_out(lw.la_a, [sp.la_v_heads])
        out.la_b = slice_out(lw.la_b, [sp.la_v_heads])
        out.la_out = slice_in(lw.la_out, *_head_rows(sp.la_v_heads, vd))
        idx = torch.cat([torch.arange(a, b) for a, b in qkv_ranges]).to(lw.la_conv1d.device)
        out.la_conv1d = lw.la_conv1d[idx].contiguous()
        a, b = sp.la_v_heads
        out.la_A_log = lw.la_A_log[a:b].contiguous()
        out.la_dt_bias = lw.la_dt_bias[a:b].contiguous()
    return out


def shard_model(mw: ModelWeights, tp_size: int, tp_rank: int) -> ModelWeights:
    cfg = mw.config
    if tp_size == 1:
        return mw
    sp = make_shard_spec(cfg, tp_size, tp_rank)
    out = ModelWeights(cfg)
    out.layers = [shard_layer(lw, cfg, tp_size, tp_rank) for lw in mw.layers]
    out.embed = mw.embed
    out.final_norm = mw.final_norm
    out.lm_head = mw.lm_head[sp.vocab[0]:sp.vocab[1]].contiguous()
    return out


def shard_weight(weight: torch.Tensor, dim: int, tp_size: int) -> List[torch.Tensor]:
    """Split a dense tensor evenly along `dim` (reference:
    src/runtime/tensor_parallel.py:336-391)."""
    if weight.shape[dim] % tp_size:
        raise ValueError("dimension not divisible by tp_size")
    return [c.contiguous() for c in weight.chunk(tp_size, dim=dim)]
