"""Communicator interface shared by every backend.

The reference's communication layer is a set of single-process, multi-device
all-reduce implementations chosen by flags (reference:
src/inference/tp_engine.py:4311-4409, src/runtime/p2p_allreduce.py,
src/runtime/tensor_parallel.py:76-334).  Here a communicator belongs to one
rank of a `torch.distributed` job:

* `SingleComm`     : tp_size == 1, every collective is the identity.
* `TorchDistComm`  : gloo on CPU (tests, host-side plumbing, the replacement of
                     the reference's host AVX all-reduce, src/runtime/fast_allreduce.c)
                     or NCCL on GPU (the in-repo baseline only).
* `SymmComm`       : (parallel/symm.py) symmetric memory over NVLink with the
                     collectives issued from inside this package's CUDA kernels.

All of them count all-reduce calls like the reference does
(reference: src/inference/tp_engine.py:2495-2501).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


class CommTimeout(RuntimeError):
    """A bounded device-side or host-side wait expired."""


class Communicator:
    tp_size: int = 1
    tp_rank: int = 0

    def __init__(self):
        self.allreduce_calls = 0

    # reference-compatible counters
    def get_allreduce_call_count(self) -> int:
        return self.allreduce_calls

    def reset_allreduce_counter(self) -> None:
        self.allreduce_calls = 0

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def all_gather(self, t: torch.Tensor) -> List[torch.Tensor]:
        raise NotImplementedError

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        raise NotImplementedError

    def scatter(self, chunks: Optional[List[torch.Tensor]], like: torch.Tensor, src: int = 0):
        raise NotImplementedError

    def gather(self, t: torch.Tensor, dst: int = 0) -> Optional[List[torch.Tensor]]:
        raise NotImplementedError

    def reduce_scatter_sum(self, t: torch.Tensor) -> torch.Tensor:
        """t[tp*n, ...] -> this rank's reduced [n, ...] slice."""
        raise NotImplementedError

    def barrier(self) -> None:
        pass

    # the fused form every residual update uses
    def allreduce_residual(self, partial: torch.Tensor, hidden: torch.Tensor) -> torch.Tensor:
        """hidden += sum over ranks of partial (reference:
        src/runtime/p2p_allreduce.py:334-429)."""
        hidden += self.all_reduce_sum(partial)
        return hidden


    def sequence_parallel_handoff(self, partial: torch.Tensor, hidden: torch.Tensor, norm_w: torch.Tensor,
                                  eps: float) -> torch.Tensor:
        """Sequence-parallel hand-off after a row-parallel projection of T rows: rank r owns rows
        [r * ceil(T / tp), ...).  hidden[own rows] += sum over ranks of partial[own rows]; returns the RMS-normalised
        rows (times norm_w) of ALL ranks, fp16.  Only the owner's rows of `hidden` are kept up to date, plus the
        last row on every rank.  This is the portable composition (reduce-scatter, local norm, all-gather); on
        GPUs `SymmComm.reduce_scatter_norm_allgather` does it in one kernel (csrc/comm.cu, rs_norm_ag_kernel)."""
        T, H = partial.shape
        tp, rank = self.tp_size, self.tp_rank
        per = -(-T // tp)
        pad = per * tp - T
        p32 = partial.float()
        if pad:
            p32 = torch.cat([p32, p32.new_zeros(pad, H)])
        mine = self.reduce_scatter_sum(p32)                              # [per, H]
        lo, hi = rank * per, min(T, (rank + 1) * per)
        xn = torch.zeros(per, H, dtype=torch.float16, device=partial.device)
        last = torch.zeros(H, dtype=torch.float32, device=partial.device)
        if lo < hi:
            hidden[lo:hi] += mine[:hi - lo].to(hidden.dtype)
            h = hidden[lo:hi].float()
            xn[:hi - lo] = (h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * norm_w.float()).half()
            if hi == T:
                last = hidden[T - 1].float().clone()
        out = torch.cat(self.all_gather(xn))[:T]
        last = self.all_reduce_sum(last)                                 # only the owner contributes
        self.allreduce_calls -= 1
        hidden[T - 1] = last.to(hidden.dtype)
        return out


class SingleComm(Communicator):
    def all_reduce_sum(self, t):
        self.allreduce_calls += 1
        return t

    def all_gather(self, t):
        return [t]

    def broadcast(self, t, src=0):
        return t

    def scatter(self, chunks, like, src=0):
        return chunks[0]

    def gather(self, t, dst=0):
        return [t]

    def reduce_scatter_sum(self, t):
        return t


class TorchDistComm(Communicator):
    """`torch.distributed` collectives on the default (or a given) group."""

    def __init__(self, group=None):
        super().__init__()
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.tp_size = dist.get_world_size(group)
        self.tp_rank = dist.get_rank(group)

    def all_reduce_sum(self, t):
        self.allreduce_calls += 1
        out = t.clone()
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
        return out

    def all_gather(self, t):
        outs = [torch.empty_like(t) for _ in range(self.tp_size)]
        dist.all_gather(outs, t.contiguous(), group=self.group)
        return outs

    def broadcast(self, t, src=0):
        dist.broadcast(t, src=src, group=self.group)
        return t

    def scatter(self, chunks, like, src=0):
        out = torch.empty_like(like)
        dist.scatter(out, chunks if self.tp_rank == src else None, src=src, group=self.group)
        return out

    def gather(self, t, dst=0):
        outs = [torch.empty_like(t) for _ in range(self.tp_size)] if self.tp_rank == dst else None
        dist.gather(t.contiguous(), outs, dst=dst, group=self.group)
        return outs

    def reduce_scatter_sum(self, t):
        n = t.shape[0] // self.tp_size
        out = torch.empty((n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        if t.device.type == "cpu":
            # gloo has no reduce_scatter: reduce everything, keep the own slice
            full = self.all_reduce_sum(t)
            self.allreduce_calls -= 1
            return full[self.tp_rank * n:(self.tp_rank + 1) * n].clone()
        dist.reduce_scatter_tensor(out, t.contiguous(), group=self.group)
        return out

    def barrier(self):
        dist.barrier(group=self.group)


def make_comm(tp_size: int = 1) -> Communicator:
    if tp_size == 1:
        return SingleComm()
    return TorchDistComm()
