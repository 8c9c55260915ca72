"""Guard bands around scratch and communication buffers (debug builds of a run).

A memory checker is not always at hand on a shared GPU, and the reference found its
races by symptom (reference: kernel headers of src/kernels/deltanet_v2.hip,
src/kernels/kernel_p2p_allreduce_rmsnorm.hip:72).  With
`EngineConfig.debug_guards` every work buffer is allocated with a poisoned band
on both sides; `check_all()` after a step reports any band a kernel wrote into,
by buffer name and offset, without any illegal access having taken place.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

POISON_BYTE = 0xA5


class GuardError(RuntimeError):
    pass


class GuardedAllocator:
    def __init__(self, device, band_bytes: int = 4096):
        self.device = torch.device(device)
        self.band = (band_bytes + 255) // 256 * 256
        self._bufs: Dict[str, Tuple[torch.Tensor, int]] = {}

    def zeros(self, name: str, shape, dtype) -> torch.Tensor:
        """A zero tensor of `shape` whose storage is preceded and followed by a poisoned band."""
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        body = (nbytes + 255) // 256 * 256
        raw = torch.full((self.band + body + self.band,), POISON_BYTE, dtype=torch.uint8, device=self.device)
        raw[self.band:self.band + nbytes] = 0
        self._bufs[name] = (raw, nbytes)
        return raw[self.band:self.band + nbytes].view(dtype).view(shape)

    def check(self, name: str) -> List[int]:
        raw, nbytes = self._bufs[name]
        lo = raw[:self.band]
        hi = raw[self.band + nbytes:]
        bad = []
        for base, part in ((0, lo), (self.band + nbytes, hi)):
            idx = torch.nonzero(part != POISON_BYTE).flatten()
            if idx.numel():
                bad.append(base + int(idx[0]) - self.band)      # byte offset relative to the buffer start
        return bad

    def check_all(self):
        problems = {n: b for n in self._bufs if (b := self.check(n))}
        if problems:
            raise GuardError("writes outside buffers (byte offsets relative to the buffer): " +
                             ", ".join(f"{n}: {b}" for n, b in problems.items()))

    def names(self) -> List[str]:
        return list(self._bufs)
