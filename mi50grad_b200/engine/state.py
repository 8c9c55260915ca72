"""Per-sequence device state: KV cache, Gated DeltaNet state, lengths.

The reference keeps a contiguous fp16 KV cache for the full-attention layers
with ONE shared length for all sequences (reference: src/inference/engine.py:79-290,
:94) and an fp32 recurrent state plus fp16 conv history per DeltaNet layer
(reference: src/inference/engine.py:293-369).  Here every sequence slot has its
own length, kept in device memory so captured graphs can read it, and the whole
position-dependent state of a slot can be snapshotted and restored -- which is
what speculative rollback and recovery need and what the reference cannot do
for its DeltaNet layers (reference: src/inference/tp_engine.py:1673-1687).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..config import QwenConfig
from ..parallel.sharding import ShardSpec

DN_COLS = 32


class KVCache:
    """[full_layers][batch][max_seq][local_kv_heads][head_dim] fp16, K and V."""

    def __init__(self, cfg: QwenConfig, spec: ShardSpec, max_seq_len: int, max_batch: int, device):
        self.layers = cfg.full_attention_layer_indices()
        self.index = {li: i for i, li in enumerate(self.layers)}
        shape = (len(self.layers), max_batch, max_seq_len, spec.n_kv, cfg.head_dim)
        self.k = torch.zeros(shape, dtype=torch.float16, device=device)
        self.v = torch.zeros(shape, dtype=torch.float16, device=device)
        self.max_seq_len = max_seq_len

    def layer_k(self, layer_idx: int) -> torch.Tensor:
        return self.k[self.index[layer_idx]]

    def layer_v(self, layer_idx: int) -> torch.Tensor:
        return self.v[self.index[layer_idx]]

    def nbytes(self) -> int:
        return 2 * self.k.numel() * 2


class DeltaNetState:
    """fp32 state [lin_layers][batch][v_heads][dk][dv]; fp16 conv history stored
    per consuming CTA: [lin_layers][batch][v_heads][dv/32][2*dk+32][3]."""

    def __init__(self, cfg: QwenConfig, spec: ShardSpec, max_batch: int, device):
        self.layers = cfg.linear_attention_layer_indices()
        self.index = {li: i for i, li in enumerate(self.layers)}
        dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.nch = 2 * dk + DN_COLS
        self.S = torch.zeros(len(self.layers), max_batch, spec.n_la_v, dk, dv, dtype=torch.float32,
                             device=device)
        self.conv = torch.zeros(len(self.layers), max_batch, spec.n_la_v, dv // DN_COLS, self.nch, 3,
                                dtype=torch.float16, device=device)

    def layer_S(self, layer_idx: int) -> torch.Tensor:
        return self.S[self.index[layer_idx]]

    def layer_conv(self, layer_idx: int) -> torch.Tensor:
        return self.conv[self.index[layer_idx]]

    def nbytes(self) -> int:
        return self.S.numel() * 4 + self.conv.numel() * 2


@dataclass
class SequenceSnapshot:
    """Device copy of everything position-dependent for one sequence slot."""
    seq: int
    length: int
    token: int
    k: Optional[torch.Tensor]
    v: Optional[torch.Tensor]
    S: torch.Tensor
    conv: torch.Tensor


class SequenceStates:
    """Lengths + caches of all slots.  `seqs` is the device array of
    {len, token, pad, pad} the kernels read."""

    def __init__(self, cfg: QwenConfig, spec: ShardSpec, max_seq_len: int, max_batch: int, device):
        self.kv = KVCache(cfg, spec, max_seq_len, max_batch, device)
        self.dn = DeltaNetState(cfg, spec, max_batch, device)
        self.seqs = torch.zeros(max_batch, 4, dtype=torch.int32, device=device)
        self.max_batch = max_batch

    def lengths(self) -> List[int]:
        return self.seqs[:, 0].tolist()

    def length(self, seq: int = 0) -> int:
        return int(self.seqs[seq, 0].item())

    def set_length(self, seq: int, n: int):
        self.seqs[seq, 0] = n

    def set_token(self, seq: int, tok: int):
        self.seqs[seq, 1] = tok

    def token(self, seq: int = 0) -> int:
        return int(self.seqs[seq, 1].item())

    def reset(self, seq: Optional[int] = None):
        if seq is None:
            self.seqs.zero_()
            self.dn.S.zero_()
            self.dn.conv.zero_()
        else:
            self.seqs[seq].zero_()
            self.dn.S[:, seq].zero_()
            self.dn.conv[:, seq].zero_()

    def snapshot(self, seq: int = 0, with_kv: bool = False) -> SequenceSnapshot:
        """KV entries beyond the snapshotted length are never visible again after
        a restore, so the cache itself only needs copying for full checkpoints."""
        n = self.length(seq)
        return SequenceSnapshot(
            seq, n, self.token(seq),
            self.kv.k[:, seq, :n].clone() if with_kv else None,
            self.kv.v[:, seq, :n].clone() if with_kv else None,
            self.dn.S[:, seq].clone(), self.dn.conv[:, seq].clone())

    def restore(self, snap: SequenceSnapshot, seq: Optional[int] = None):
        seq = snap.seq if seq is None else seq
        self.seqs[seq, 0] = snap.length
        self.seqs[seq, 1] = snap.token
        self.dn.S[:, seq].copy_(snap.S)
        self.dn.conv[:, seq].copy_(snap.conv)
        if snap.k is not None:
            self.kv.k[:, seq, :snap.length].copy_(snap.k)
            self.kv.v[:, seq, :snap.length].copy_(snap.v)

    def state_dict(self, seq: int = 0) -> Dict[str, torch.Tensor]:
        """Host-serialisable checkpoint of one sequence."""
        s = self.snapshot(seq, with_kv=True)
        return {"length": torch.tensor(s.length), "token": torch.tensor(s.token), "k": s.k.cpu(),
                "v": s.v.cpu(), "S": s.S.cpu(), "conv": s.conv.cpu()}

    def load_state_dict(self, sd: Dict[str, torch.Tensor], seq: int = 0):
        dev = self.seqs.device
        self.restore(SequenceSnapshot(seq, int(sd["length"]), int(sd["token"]), sd["k"].to(dev),
                                      sd["v"].to(dev), sd["S"].to(dev), sd["conv"].to(dev)), seq)
