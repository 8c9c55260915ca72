"""Symmetric-memory communicator over NVLink / NVSwitch.

Every rank allocates the same buffers through PyTorch's symmetric-memory
allocator (CUDA VMM allocations whose handles are exchanged once at rendezvous),
maps all peers' copies, and -- when the fabric offers it -- gets a multicast
mapping so kernels can issue `multimem.ld_reduce` / `multimem.st`.  PyTorch does
the allocation and the handle exchange; every byte that moves afterwards is
moved by this package's kernels (csrc/gemv.cu finisher, csrc/comm.cu).

Replaces the reference's single-process peer plumbing: `hipDeviceEnablePeerAccess`
between all pairs, gather buffers on GPU 0, per-GPU all-reduce streams and
host-recorded events (reference: src/runtime/tensor_parallel.py:47-58,
src/runtime/p2p_allreduce.py:73-104, :257-332).

Layout of the symmetric block (bytes):
    [0, 2*part_floats*4)            partial-sum staging, double-buffered by epoch parity
    [+0, +gather_floats*4)          two-shot gather area
    [.., +256)                      flag words: [0,8) phase A, [8,16) phase B (uint32, by source rank)
    [.., +2*tp*8*tile_h*8)          tile staging of the chain kernel: [parity][source rank][row][tile_h] {fp32, epoch}
    [.., +8*TILE_FLAGS*4)           tile flags: [source rank][tile] uint32
    [.., +part_floats*2)            fp16 activations of many-row steps, all-gathered by rs_norm_ag_kernel
    [.., +hidden*4)                 fp32 residual of the last row of such a step
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import lib as L
from .comm import CommTimeout, Communicator

class SeqParParams(C.Structure):
    _fields_ = [("comm", L.CommCtx), ("h", C.c_void_p), ("norm_w", C.c_void_p), ("xn", C.c_void_p * L.MAX_TP),
                ("mc_xn", C.c_void_p), ("hlast", C.c_void_p * L.MAX_TP), ("T", C.c_int), ("H", C.c_int),
                ("rows_per", C.c_int), ("eps", C.c_float), ("counters", C.c_void_p), ("test_withhold", C.c_int),
                ("pad", C.c_int)]


KERNEL_NAMES = {1: "gemv finisher", 2: "all-reduce", 3: "arg-max", 4: "barrier", 5: "wait self-test", 6: "gemm reduce-scatter",
                7: "chain dependency", 8: "chain tile exchange", 9: "chain weight copy", 10: "distributed sampler", 11: "reduce-scatter + norm + all-gather"}


class CollParams(C.Structure):
    _fields_ = [("comm", L.CommCtx), ("in_", C.c_void_p), ("in16", C.c_void_p), ("out", C.c_void_p),
                ("out16", C.c_void_p), ("gather", C.c_void_p * L.MAX_TP), ("mc_gather", C.c_void_p),
                ("n", C.c_size_t), ("residual", C.c_int), ("twoshot", C.c_int), ("counters", C.c_void_p),
                ("test_withhold", C.c_int), ("pushed", C.c_int)]


class SymmComm(Communicator):
    def __init__(self, max_rows: int = 8, hidden: int = 5120, part_floats: Optional[int] = None,
                 use_multimem: bool = True, wait_us: int = 2_000_000, group=None):
        super().__init__()
        import torch.distributed._symmetric_memory as symm_mem
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group or dist.group.WORLD
        self.tp_size, self.tp_rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.tp_size > L.MAX_TP:
            raise ValueError(f"at most {L.MAX_TP} ranks")
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.lib = L.lib()
        if self.lib.b2_sizeof_coll_params() != C.sizeof(CollParams):
            raise RuntimeError("CollParams layout mismatch")
        self.part_floats = int(part_floats or max(max_rows * hidden, 4096))
        self.part_floats = -(-self.part_floats // 64) * 64
        self.gather_floats = self.part_floats
        self.off_gather = 2 * self.part_floats * 4
        self.off_sig = self.off_gather + self.gather_floats * 4
        # tile-granular exchange of the persistent chain kernel (csrc/chain.cu)
        self.tile_h = -(-int(hidden) // 64) * 64
        self.tile_flags = max(128, self.tile_h // 64)
        self.off_tpart = self.off_sig + 256
        self.off_tsig = self.off_tpart + 2 * self.tp_size * L.MAX_ROWS * self.tile_h * 8      # {value, epoch} pairs
        # sequence-parallel many-row steps (csrc/comm.cu, rs_norm_ag_kernel)
        self.off_xn = -(-(self.off_tsig + L.MAX_TP * self.tile_flags * 4) // 1024) * 1024
        self.xn_halves = self.part_floats
        self.off_hlast = self.off_xn + -(-self.xn_halves * 2 // 256) * 256
        nbytes = self.off_hlast + self.tile_h * 4
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        self.hdl = symm_mem.rendezvous(self.buf, self.group)
        self.peer_ptrs: List[int] = [int(p) for p in self.hdl.buffer_ptrs]
        mc = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        self.multicast_ptr = mc if use_multimem else 0
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.counters = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.trace = torch.zeros(8, dtype=torch.int64, device=self.device)
        self.trace_enabled = False
        self.wait_ns = int(wait_us) * 1000
        torch.cuda.synchronize()
        dist.barrier(self.group)

    # -- what kernels see -------------------------------------------------------
    def ctx(self) -> L.CommCtx:
        c = L.CommCtx()
        c.tp, c.rank, c.part_stride = self.tp_size, self.tp_rank, self.part_floats
        for r in range(self.tp_size):
            c.part[r] = self.peer_ptrs[r]
            c.sig[r] = self.peer_ptrs[r] + self.off_sig
            c.tpart[r] = self.peer_ptrs[r] + self.off_tpart
            c.tsig[r] = self.peer_ptrs[r] + self.off_tsig
        c.tile_h, c.tile_flags = self.tile_h, self.tile_flags
        c.mc_part = self.multicast_ptr or None
        c.epoch, c.status, c.wait_ns = self.epoch.data_ptr(), self.status.data_ptr(), self.wait_ns
        c.trace = self.trace.data_ptr() if self.trace_enabled else None
        return c

    def xn_view(self, rows: int, hidden: int) -> torch.Tensor:
        """This rank's copy of the symmetric fp16 activation buffer of many-row steps, as a [rows, hidden] tensor."""
        if rows * hidden > self.xn_halves:
            raise ValueError(f"{rows} x {hidden} activations do not fit the symmetric buffer ({self.xn_halves} halves)")
        return self.buf[self.off_xn:self.off_xn + rows * hidden * 2].view(torch.float16).view(rows, hidden)

    def reduce_scatter_norm_allgather(self, h: torch.Tensor, norm_w: torch.Tensor, T: int, eps: float,
                                      withhold_signal: bool = False) -> torch.Tensor:
        """After every rank stored its partial rows into the owners' staging buffers (row-aligned slices of
        ceil(T / tp) rows, as the GEMM epilogue does): h[own rows] += sum of partials, normalised fp16 rows of
        every rank gathered into xn_view() on every rank.  One kernel (csrc/comm.cu, rs_norm_ag_kernel)."""
        H = h.shape[1]
        p = SeqParParams()
        p.comm = self.ctx()
        p.h, p.norm_w = h.data_ptr(), norm_w.data_ptr()
        for r in range(self.tp_size):
            p.xn[r] = self.peer_ptrs[r] + self.off_xn
            p.hlast[r] = self.peer_ptrs[r] + self.off_hlast
        p.mc_xn = (self.multicast_ptr + self.off_xn) if self.multicast_ptr else None
        p.T, p.H, p.rows_per, p.eps = T, H, -(-T // self.tp_size), eps
        p.counters, p.test_withhold = self.counters.data_ptr(), int(withhold_signal)
        L.check(self.lib.b2_rs_norm_ag(C.byref(p), L.stream()), "rs_norm_ag")
        return self.xn_view(T, H)

    def push_rows(self, partial: torch.Tensor):
        """Test helper: store this rank's [T, H] fp32 partial rows where the GEMM epilogue would have stored
        them (the staging buffer of each row's owner, parity of the next epoch)."""
        T, H = partial.shape
        per = -(-T // self.tp_size)
        parity = (int(self.epoch.item()) + 1) & 1
        for r in range(self.tp_size):
            lo, hi = r * per, min(T, (r + 1) * per)
            if lo >= hi:
                continue
            dst = self.hdl.get_buffer(r, (per * H,), torch.float32,
                                      parity * self.part_floats + self.tp_rank * per * H)
            dst[:(hi - lo) * H].copy_(partial[lo:hi].reshape(-1))
        torch.cuda.synchronize()

    def last_exchange_trace(self) -> dict:
        """globaltimer stamps (ns) of the last fused GEMV exchange on this rank, relative to the
        kernel's start: entry of the finishing CTA, flags of all peers seen, residual+sums done."""
        t = self.trace.tolist()
        return {"finisher_entry_ns": t[0] - t[3], "peers_arrived_ns": t[1] - t[3], "reduced_ns": t[2] - t[3]}

    @property
    def has_multimem(self) -> bool:
        return bool(self.multicast_ptr)

    def check_status(self):
        """Raise CommTimeout if any kernel's bounded wait expired since the last check."""
        st = self.status.tolist()
        if st[0] != 0:
            self.status.zero_()
            raise CommTimeout(f"rank {self.tp_rank}: bounded wait expired in {KERNEL_NAMES.get(st[1], st[1])} "
                              f"waiting for rank {st[2]} at epoch {st[3]}")

    # -- collectives --------------------------------------------------------------
    def _params(self, n: int, residual: bool, twoshot: bool) -> CollParams:
        p = CollParams()
        p.comm = self.ctx()
        for r in range(self.tp_size):
            p.gather[r] = self.peer_ptrs[r] + self.off_gather
        p.mc_gather = (self.multicast_ptr + self.off_gather) if self.multicast_ptr else None
        p.n, p.residual, p.twoshot = n, int(residual), int(twoshot)
        p.counters = self.counters.data_ptr()
        return p

    def all_reduce_into(self, src: torch.Tensor, out: torch.Tensor, residual: bool = False,
                        twoshot: Optional[bool] = None, out16: Optional[torch.Tensor] = None,
                        withhold_signal: bool = False) -> torch.Tensor:
        """out (fp32) = [out +] sum over ranks of src (fp32 or fp16), in one kernel."""
        n = src.numel()
        if n % 4 or n > self.part_floats:
            raise ValueError(f"payload of {n} elements: need a multiple of 4 and <= {self.part_floats}")
        if twoshot is None:
            twoshot = n * 4 > 512 * 1024
        p = self._params(n, residual, twoshot)
        if src.dtype == torch.float32:
            p.in_ = src.data_ptr()
        elif src.dtype == torch.float16:
            p.in16 = src.data_ptr()
        else:
            raise TypeError("fp32 or fp16 input")
        p.out = out.data_ptr()
        p.out16 = None if out16 is None else out16.data_ptr()
        p.test_withhold = int(withhold_signal)
        L.check(self.lib.b2_allreduce(C.byref(p), 2 * 148, L.stream()), "allreduce")
        self.allreduce_calls += 1
        return out

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        out = torch.empty(t.shape, dtype=torch.float32, device=t.device)
        self.all_reduce_into(t.contiguous(), out)
        return out if t.dtype == torch.float32 else out.to(t.dtype)

    def allreduce_residual(self, partial: torch.Tensor, hidden: torch.Tensor) -> torch.Tensor:
        return self.all_reduce_into(partial.contiguous(), hidden, residual=True)

    def device_barrier(self, withhold_signal: bool = False):
        c = self.ctx()
        L.check(self.lib.b2_barrier(C.byref(c), int(withhold_signal), L.stream()), "barrier")

    def barrier(self):
        self.device_barrier()

    def all_gather(self, t):
        outs = [torch.empty_like(t) for _ in range(self.tp_size)]
        dist.all_gather(outs, t.contiguous(), group=self.group)
        return outs

    def broadcast(self, t, src=0):
        dist.broadcast(t, src=src, group=self.group)
        return t

    def close(self):
        self.buf = None
        self.hdl = None
