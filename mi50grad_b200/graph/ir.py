"""Small operator-graph IR of the decode step.

The reference ships an unused IR with a placeholder `toposort`
(src/graph/ir.py:1-111).  Here the IR is used for accounting: `build_layer_graph`
/ `build_step_graph` describe the step the C++ driver issues (one node per kernel
launch, edges = data dependencies), `toposort` is a real Kahn sort, and
`Graph.summary()` gives launches, weight bytes and FLOPs per step, which the
benchmark prints next to its measurements.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, List, Optional, Sequence, Tuple


class DType(Enum):
    F32 = "f32"
    F16 = "f16"
    BF16 = "bf16"
    I32 = "i32"
    I8 = "i8"
    I4 = "i4"

    @property
    def itemsize(self) -> float:
        return {"f32": 4, "f16": 2, "bf16": 2, "i32": 4, "i8": 1, "i4": 0.5}[self.value]


@dataclass
class TensorInfo:
    name: str
    shape: Tuple[int, ...]
    dtype: DType = DType.F16

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= int(s)
        return n

    @property
    def nbytes(self) -> int:
        return int(self.numel * self.dtype.itemsize)


class OpType(Enum):
    EMBED_RMSNORM = "embed_rmsnorm"
    GEMV_INT4 = "gemv_int4"
    GEMV_INT4_SILU = "gemv_int4_silu_pair"
    GEMV_INT4_FINISH = "gemv_int4_allreduce_residual"
    GEMV_F16 = "gemv_f16"
    QKNORM_ROPE_CACHEW = "qknorm_rope_cachew"
    DECODE_ATTN = "decode_attn"
    DELTANET_STEP = "deltanet_step"
    ARGMAX = "argmax"
    ADVANCE = "advance"
    PREPARE_ROWS = "prepare_rows"


@dataclass
class Op:
    type: OpType
    name: str
    inputs: List[str] = field(default_factory=list)
    outputs: List[str] = field(default_factory=list)
    weight_bytes: int = 0
    flops: int = 0
    collective: Optional[str] = None       # "all_reduce" when the kernel exchanges partials itself
    attrs: Dict[str, object] = field(default_factory=dict)


class Graph:
    def __init__(self, name: str = "step"):
        self.name = name
        self.ops: List[Op] = []
        self.tensors: Dict[str, TensorInfo] = {}

    def add_tensor(self, t: TensorInfo) -> TensorInfo:
        self.tensors[t.name] = t
        return t

    def add_op(self, op: Op) -> Op:
        self.ops.append(op)
        return op

    def toposort(self) -> List[Op]:
        """Kahn's algorithm over producer -> consumer edges; among ready ops the
        insertion order is kept.  A tensor written more than once (the residual
        stream) orders its writers and readers by insertion order."""
        last_writer: Dict[str, int] = {}
        readers_since: Dict[str, List[int]] = {}
        deps: List[set] = [set() for _ in self.ops]
        for i, op in enumerate(self.ops):
            for t in op.inputs:
                if t in last_writer:
                    deps[i].add(last_writer[t])
                readers_since.setdefault(t, []).append(i)
            for t in op.outputs:
                if t in last_writer:
                    deps[i].add(last_writer[t])
                for r in readers_since.get(t, []):
                    if r != i:
                        deps[i].add(r)
                last_writer[t] = i
                readers_since[t] = []
        indeg = [len(d) for d in deps]
        users: List[List[int]] = [[] for _ in self.ops]
        for i, d in enumerate(deps):
            for j in d:
                users[j].append(i)
        ready = [i for i, n in enumerate(indeg) if n == 0]
        order: List[Op] = []
        while ready:
            ready.sort()
            i = ready.pop(0)
            order.append(self.ops[i])
            for u in users[i]:
                indeg[u] -= 1
                if indeg[u] == 0:
                    ready.append(u)
        if len(order) != len(self.ops):
            raise ValueError("cycle in graph")
        return order

    def summary(self) -> Dict[str, float]:
        return {"launches": len(self.ops), "weight_bytes": sum(o.weight_bytes for o in self.ops),
                "flops": sum(o.flops for o in self.ops),
                "collectives": sum(1 for o in self.ops if o.collective)}


def _int4_bytes(K: int, N: int, group: int) -> int:
    return K * N // 2 + (K // group) * N * 4


def build_layer_graph(g: Graph, cfg, spec, li: int, rows: int = 1, ar_mode: str = "exact") -> None:
    """Append the launches of layer `li` (same sequence as csrc/driver.cu)."""
    H, gs = cfg.hidden_size, cfg.group_size
    tp = spec.tp_size
    p = f"l{li}."
    if cfg.is_full_attention(li):
        qd, kvd = spec.n_q * cfg.head_dim, spec.n_kv * cfg.head_dim
        n_in, k_out = 2 * qd + 2 * kvd, qd
    else:
        kd, vd = spec.n_la_k * cfg.linear_key_head_dim, spec.n_la_v * cfg.linear_value_head_dim
        n_in, k_out = 2 * kd + 2 * vd, vd
    g.add_op(Op(OpType.GEMV_INT4, p + "in_proj", ["h", "ss"], [p + "proj"], _int4_bytes(H, n_in, gs), 2 * rows * H * n_in))
    if cfg.is_full_attention(li):
        g.add_op(Op(OpType.QKNORM_ROPE_CACHEW, p + "qknorm_rope", [p + "proj", "rows"], [p + "proj", p + "kv"]))
        g.add_op(Op(OpType.DECODE_ATTN, p + "attn", [p + "proj", p + "kv", "rows"], [p + "attn_out"]))
    else:
        g.add_op(Op(OpType.DELTANET_STEP, p + "deltanet", [p + "proj", "h", "ss", "rows"], [p + "attn_out", p + "state"]))
    coll_attn = "all_reduce" if tp > 1 and ar_mode == "exact" else None
    g.add_op(Op(OpType.GEMV_INT4_FINISH, p + "out_proj", [p + "attn_out", "h"], ["h", "ss"],
                _int4_bytes(k_out, H, gs), 2 * rows * k_out * H, coll_attn))
    F = spec.ffn_local
    g.add_op(Op(OpType.GEMV_INT4_SILU, p + "gate_up", ["h", "ss"], [p + "act"], _int4_bytes(H, 2 * F, gs), 4 * rows * H * F))
    g.add_op(Op(OpType.GEMV_INT4_FINISH, p + "down", [p + "act", "h"], ["h", "ss"], _int4_bytes(F, H, gs),
                2 * rows * F * H, "all_reduce" if tp > 1 else None))


def build_step_graph(cfg, spec, rows: int = 1, ar_mode: str = "exact") -> Graph:
    g = Graph("decode_step")
    g.add_op(Op(OpType.PREPARE_ROWS, "prepare_rows", ["rows_tmpl", "seqs"], ["rows"]))
    g.add_op(Op(OpType.EMBED_RMSNORM, "embed", ["tokens", "rows"], ["h", "ss"]))
    for li in range(cfg.num_hidden_layers):
        build_layer_graph(g, cfg, spec, li, rows, ar_mode)
    g.add_op(Op(OpType.GEMV_F16, "lm_head", ["h", "ss"], ["logits"], spec.vocab_local * cfg.hidden_size * 2,
                2 * rows * spec.vocab_local * cfg.hidden_size))
    g.add_op(Op(OpType.ARGMAX, "argmax", ["logits"], ["out_tokens", "seqs"],
                collective="all_gather" if spec.tp_size > 1 else None))
    g.add_op(Op(OpType.ADVANCE, "advance", ["seqs"], ["seqs"]))
    return g
