"""Run metrics, logging and phase timing.

The reference prints from everywhere and times steps with `time.perf_counter`
after a device sync (reference: src/inference/generate.py:205-236,
tests/bench_pp_tg.py:112-118,283-296).  Here a run fills one `Metrics` record
(throughput, step time, exposed communication, collective and launch counts,
speculation acceptance) that is dumped as one JSON object, messages go through
`logging`, and `PhaseTimer` brackets named phases with CUDA events (plus NVTX
ranges when a profiler wants them) without synchronising inside the phase.
"""
from __future__ import annotations

import json
import logging
import time
from contextlib import contextmanager
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional


def get_logger(name: str = "mi50grad_b200", level: int = logging.INFO) -> logging.Logger:
    log = logging.getLogger(name)
    if not log.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter("%(asctime)s %(name)s %(levelname)s %(message)s"))
        log.addHandler(h)
        log.setLevel(level)
        log.propagate = False
    return log


@dataclass
class Metrics:
    run: str = ""
    n_gpus: int = 1
    tokens: int = 0
    steps: int = 0
    seconds: float = 0.0
    ms_per_step: float = 0.0
    tok_per_s: float = 0.0
    prefill_tokens: int = 0
    prefill_ms: float = 0.0
    ttft_ms: float = 0.0
    exposed_comm_us_per_step: Optional[float] = None
    allreduce_calls: int = 0
    launches_per_step: int = 0
    drafted: int = 0
    accepted: int = 0
    phases_ms: Dict[str, float] = field(default_factory=dict)
    extra: Dict[str, object] = field(default_factory=dict)

    def finish(self) -> "Metrics":
        if self.steps and self.seconds > 0:
            self.ms_per_step = 1e3 * self.seconds / self.steps
        if self.tokens and self.seconds > 0:
            self.tok_per_s = self.tokens / self.seconds
        return self

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.drafted if self.drafted else 0.0

    def to_dict(self) -> dict:
        d = asdict(self)
        d["acceptance_rate"] = self.acceptance_rate
        return d

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), sort_keys=True)

    def dump(self, path: str):
        with open(path, "a", encoding="utf-8") as f:
            f.write(self.to_json() + "\n")


class PhaseTimer:
    """Named phases timed on the device.  `with timer.phase("prefill"): ...` records two CUDA
    events on the current stream (host clock when CUDA is absent); `summary()` synchronises once
    and returns milliseconds per phase (summed over repeats)."""

    def __init__(self, use_cuda: Optional[bool] = None, nvtx: bool = False):
        import torch
        self._torch = torch
        self.cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self.nvtx = nvtx and self.cuda
        self._pairs: List[tuple] = []
        self._host: Dict[str, float] = {}

    @contextmanager
    def phase(self, name: str):
        torch = self._torch
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if self.nvtx:
                torch.cuda.nvtx.range_push(name)
            a.record()
            try:
                yield
            finally:
                b.record()
                if self.nvtx:
                    torch.cuda.nvtx.range_pop()
                self._pairs.append((name, a, b))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._host[name] = self._host.get(name, 0.0) + 1e3 * (time.perf_counter() - t0)

    def summary(self) -> Dict[str, float]:
        out = dict(self._host)
        if self.cuda and self._pairs:
            self._torch.cuda.synchronize()
            for name, a, b in self._pairs:
                out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out
