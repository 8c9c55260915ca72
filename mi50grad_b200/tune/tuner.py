"""Launch-shape tuning database and sweep helper.

`TuneConfig` / `TuneResult` / `TuneDB` keep the reference's names (its tuner is an
unused stub: src/tune/tuner.py:1-93).  Here the database is used: `sweep()` times
candidate configurations of an op with CUDA events inside a captured graph and
stores the best one keyed by (op, M, N, K, dtype, device name); `ops.packing`
can be pointed at a database to override its launch-shape heuristic.
"""
from __future__ import annotations

import json
import sqlite3
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional


@dataclass(frozen=True)
class TuneConfig:
    """One candidate: free-form integer parameters (k_splits, L, stages, t_tile, ...)."""
    params: tuple = ()

    @classmethod
    def of(cls, **kw: int) -> "TuneConfig":
        return cls(tuple(sorted((k, int(v)) for k, v in kw.items())))

    def as_dict(self) -> Dict[str, int]:
        return dict(self.params)

    def key(self) -> str:
        return json.dumps(self.as_dict(), sort_keys=True)


@dataclass
class TuneResult:
    config: TuneConfig
    time_us: float
    gbytes_per_s: float = 0.0
    tflops: float = 0.0
    device: str = ""
    stamp: float = field(default_factory=time.time)


class TuneDB:
    def __init__(self, db_path: str = "tune.db"):
        self.path = db_path
        self.conn = sqlite3.connect(db_path)
        self._init_db()

    def _init_db(self):
        self.conn.execute(
            "CREATE TABLE IF NOT EXISTS results (op TEXT, m INTEGER, n INTEGER, k INTEGER, dtype TEXT, device TEXT,"
            " config TEXT, time_us REAL, gbs REAL, tflops REAL, stamp REAL,"
            " PRIMARY KEY (op, m, n, k, dtype, device, config))")
        self.conn.commit()

    def store(self, op: str, m: int, n: int, k: int, dtype: str, result: TuneResult):
        self.conn.execute("INSERT OR REPLACE INTO results VALUES (?,?,?,?,?,?,?,?,?,?,?)",
                          (op, m, n, k, dtype, result.device, result.config.key(), result.time_us,
                           result.gbytes_per_s, result.tflops, result.stamp))
        self.conn.commit()

    def best(self, op: str, m: int, n: int, k: int, dtype: str, device: Optional[str] = None) -> Optional[TuneResult]:
        q = "SELECT config, time_us, gbs, tflops, device, stamp FROM results WHERE op=? AND m=? AND n=? AND k=? AND dtype=?"
        args: List[Any] = [op, m, n, k, dtype]
        if device is not None:
            q += " AND device=?"
            args.append(device)
        row = self.conn.execute(q + " ORDER BY time_us ASC LIMIT 1", args).fetchone()
        if row is None:
            return None
        return TuneResult(TuneConfig.of(**json.loads(row[0])), row[1], row[2], row[3], row[4], row[5])

    def all(self, op: Optional[str] = None) -> List[tuple]:
        if op is None:
            return self.conn.execute("SELECT * FROM results ORDER BY op, m, n, k, time_us").fetchall()
        return self.conn.execute("SELECT * FROM results WHERE op=? ORDER BY m, n, k, time_us", (op,)).fetchall()

    def close(self):
        self.conn.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def sweep(op: str, m: int, n: int, k: int, dtype: str, candidates: Iterable[TuneConfig],
          run: Callable[[TuneConfig], float], db: Optional[TuneDB] = None, bytes_moved: float = 0.0,
          flops: float = 0.0, device: str = "") -> Optional[TuneResult]:
    """`run(config)` returns microseconds (or raises / returns inf for an invalid
    configuration).  Every valid result is stored; the best is returned."""
    best: Optional[TuneResult] = None
    for cfg in candidates:
        try:
            us = float(run(cfg))
        except (ValueError, RuntimeError):
            continue
        if not us > 0 or us == float("inf"):
            continue
        r = TuneResult(cfg, us, bytes_moved / us / 1e3 if bytes_moved else 0.0, flops / us / 1e6 if flops else 0.0, device)
        if db is not None:
            db.store(op, m, n, k, dtype, r)
        if best is None or us < best.time_us:
            best = r
    return best


def time_graph_us(fn: Callable[[], None], iters: int = 20, warmup: int = 3) -> float:
    """Mean device time of fn() in microseconds: `iters` calls captured into one
    CUDA graph, replayed after warm-up, bracketed by events."""
    import torch
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for _ in range(iters):
                fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters
