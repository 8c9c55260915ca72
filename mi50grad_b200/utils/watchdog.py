"""Host-side failure detection and recovery for a tensor-parallel run.

The reference has neither (errors are return codes; device waits are unbounded:
src/kernels/gemv_int4_p2p_allreduce_rmsnorm.hip:322-325).  Three pieces, all on
the host so that nothing ever has to fault a GPU:

* `Heartbeat`: every rank publishes (step, wall time) under its own key of a
  key-value store (the torch.distributed store of the bootstrap, or any object
  with set/get) from a small thread and at step boundaries;
* `Watchdog.check()`: before launching the next step a rank looks at its peers'
  heartbeats and failure marks and raises `RankFailure(rank, reason)` instead of
  entering a collective that cannot complete.  Together with the kernels' bounded
  waits (`CommTimeout`) this bounds the time to detection from both sides;
* `recover()`: tear the process group down, bootstrap a new one (same or smaller
  world) and restore every sequence from its last snapshot.
"""
from __future__ import annotations

import json
import threading
import time
from typing import Callable, Dict, List, Optional


class RankFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class DictStore:
    """In-process stand-in for a distributed store (tests, single process)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, k: str, v):
        with self._lock:
            self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        with self._lock:
            return self._d[k]

    def check(self, keys) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


def _has(store, key: str) -> bool:
    chk = getattr(store, "check", None)
    if chk is not None:
        return bool(chk([key]))
    try:
        store.get(key)
        return True
    except Exception:
        return False


class Heartbeat:
    def __init__(self, store, rank: int, prefix: str = "hb", interval_s: float = 0.2, clock: Callable[[], float] = time.time):
        self.store, self.rank, self.prefix, self.interval, self.clock = store, rank, prefix, interval_s, clock
        self.step = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def key(self, rank: Optional[int] = None) -> str:
        return f"{self.prefix}/{self.rank if rank is None else rank}"

    def beat(self, step: Optional[int] = None):
        if step is not None:
            self.step = step
        self.store.set(self.key(), json.dumps({"step": self.step, "t": self.clock()}))

    def mark_failed(self, reason: str):
        self.store.set(f"{self.prefix}/failed/{self.rank}", reason or "failed")

    def clear_failed(self):
        """After a recovery: withdraw this rank's failure mark (an empty mark counts as none)."""
        self.store.set(f"{self.prefix}/failed/{self.rank}", "")

    def start(self):
        self.beat()
        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:
                    return
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)


class Watchdog:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 2.0, prefix: str = "hb",
                 clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world, self.timeout, self.prefix, self.clock = store, rank, world, timeout_s, prefix, clock

    def peer_state(self, r: int) -> Optional[dict]:
        k = f"{self.prefix}/{r}"
        if not _has(self.store, k):
            return None
        return json.loads(bytes(self.store.get(k)).decode())

    def check(self, require_present: bool = True):
        """Raise RankFailure for the first peer that marked itself failed, never reported (unless
        `require_present` is off: a peer that is still starting), or whose heartbeat is older than
        the timeout."""
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            fk = f"{self.prefix}/failed/{r}"
            if _has(self.store, fk):
                why = bytes(self.store.get(fk)).decode()
                if why:
                    raise RankFailure(r, "reported failure: " + why)
            st = self.peer_state(r)
            if st is None:
                if require_present:
                    raise RankFailure(r, "no heartbeat")
                continue
            if now - st["t"] > self.timeout:
                raise RankFailure(r, f"heartbeat {now - st['t']:.1f} s old (step {st['step']})")

    def wait_for_step(self, step: int, poll_s: float = 0.01):
        """Block until every peer reports `step` or later; RankFailure if one cannot."""
        t0 = self.clock()
        at = lambda r: (self.peer_state(r) or {"step": -1})["step"]
        while True:
            self.check(require_present=False)                  # a peer may still be starting up
            if all(at(r) >= step for r in range(self.world) if r != self.rank):
                return
            if self.clock() - t0 > self.timeout:
                lag = [r for r in range(self.world) if r != self.rank and at(r) < step]
                raise RankFailure(lag[0], f"did not reach step {step} within {self.timeout} s")
            time.sleep(poll_s)


def recover(rebootstrap: Callable[[], object], restore: Callable[[object], None], snapshots) -> object:
    """Generic form: `rebootstrap()` destroys the old communicator / process group and returns a new one
    (the caller decides the new world); `restore(snapshot)` puts one sequence back (KV cache lengths,
    DeltaNet state, conv history, position).  Returns the new communicator.  The tensor-parallel engine's
    own `TPInferenceEngine.recover(snapshots)` is this with both callables filled in: a new
    symmetric-memory communicator, a rebuilt step driver, `SequenceStates.restore`."""
    comm = rebootstrap()
    for s in snapshots:
        restore(s)
    return comm


def run_guarded(engine, fn: Callable[[], object], snapshots, retries: int = 1):
    """Run `fn()` (some steps of a TPInferenceEngine with failure detection on); if an exchange fails
    (CommTimeout) or a peer is reported down (RankFailure), recover the engine from `snapshots` and try
    again, up to `retries` times.  Every rank must take the same path: the failure is published through
    the heartbeat store, so the peers' next step boundary raises too."""
    from ..parallel.comm import CommTimeout
    for attempt in range(retries + 1):
        try:
            out = fn()
            engine.synchronize()
            engine.check_status()
            return out
        except (CommTimeout, RankFailure):
            if attempt == retries:
                raise
            engine.recover(snapshots)
