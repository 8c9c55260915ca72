"""Sweep the launch shape (CTAs along K, k-blocks per warp) of the INT4 GEMV for a model's
projection shapes and store the results in a TuneDB.

    python -m mi50grad_b200.tune.autotune --db tune.db --tp 1
    B200GRAD_TUNE_DB=tune.db python bench.py          # ops.packing then prefers the stored shapes

Timing: every candidate is replayed from a CUDA graph over three rotated weight copies (so each
launch streams from DRAM), CUDA events around the replay.
"""
from __future__ import annotations

import argparse

import torch

from ..config import qwen35_27b, tiny_config
from ..ops import kernels as K
from ..ops import lib as L
from ..ops.packing import GEMV_WK, launch_shape, random_packed_int4
from ..parallel.sharding import make_shard_spec
from .tuner import TuneConfig, TuneDB, sweep, time_graph_us


def model_gemv_shapes(cfg, tp: int):
    sp = make_shard_spec(cfg, tp, 0)
    H = cfg.hidden_size
    qd, kvd = sp.n_q * cfg.head_dim, sp.n_kv * cfg.head_dim
    kd, vd = sp.n_la_k * cfg.linear_key_head_dim, sp.n_la_v * cfg.linear_value_head_dim
    F = -(-sp.ffn_local // 64) * 64
    return {
        "attn_in_proj": (H, 2 * qd + 2 * kvd, L.EPI_STORE_F16),
        "attn_out_proj": (qd, H, L.EPI_STORE_F32),
        "deltanet_in_proj": (H, 2 * kd + 2 * vd, L.EPI_STORE_F16),
        "deltanet_out_proj": (vd, H, L.EPI_STORE_F32),
        "ffn_gate_up": (H, 2 * F, L.EPI_SILU_PAIR),
        "ffn_down": (F, H, L.EPI_STORE_F32),
    }


def candidates(KB: int, NTL: int, rows: int = 1):
    base_ks, base_L = launch_shape(KB, NTL, rows)
    seen = set()
    for ks in sorted({1, 2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16, base_ks, base_ks + 1, max(1, base_ks - 1)}):
        Lb = -(-KB // (GEMV_WK * ks))
        Lb += Lb & 1 if KB >= 2 * GEMV_WK else 0
        if Lb < 1 or 2 * GEMV_WK * Lb * (rows + 1) * 64 > 32_000:
            continue
        ks_eff = -(-KB // (GEMV_WK * Lb))
        if (ks_eff, Lb) in seen:
            continue
        seen.add((ks_eff, Lb))
        yield TuneConfig.of(k_splits=ks_eff, L=Lb)


def tune_shape(name, Kd, N, mode, db, group=128, rows=1):
    dev = torch.device("cuda")
    pks = [random_packed_int4(Kd, N, group, dev) for _ in range(3)]
    x = torch.randn(rows, Kd, device=dev).half()
    out = torch.zeros(rows, pks[0].n_pad, dtype=torch.float16 if mode != L.EPI_STORE_F32 else torch.float32, device=dev)
    scratch = torch.zeros(16 * rows * pks[0].n_pad + 4, dtype=torch.float32, device=dev)
    counters = torch.zeros(8192, dtype=torch.int32, device=dev)
    state = {"i": 0}

    def run(cfg: TuneConfig) -> float:
        d = cfg.as_dict()
        def once():
            K.gemv(pks[state["i"] % 3], x, out=out, mode=mode, scratch=scratch, counters=counters,
                   k_splits=d["k_splits"], Lblocks=d["L"])
            state["i"] += 1
        return time_graph_us(once, iters=12)
    best = sweep("gemv_int4", rows, N, Kd, "int4g%d" % group, candidates(pks[0].KB, pks[0].NTL, rows), run, db,
                 bytes_moved=pks[0].nbytes(), device=torch.cuda.get_device_name())
    base = launch_shape(pks[0].KB, pks[0].NTL, rows)
    print(f"{name:18s} K={Kd:6d} N={N:6d} heuristic (ks,L)={base} best={best.config.as_dict()} "
          f"{best.time_us:.1f} us {best.gbytes_per_s:.0f} GB/s", flush=True)
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--db", default="tune.db")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--model", default="27b", choices=["27b", "tiny"])
    a = ap.parse_args()
    cfg = qwen35_27b() if a.model == "27b" else tiny_config()
    with TuneDB(a.db) as db:
        for name, (Kd, N, mode) in model_gemv_shapes(cfg, a.tp).items():
            tune_shape(name, Kd, N, mode, db, cfg.group_size)
            for row in db.all("gemv_int4"):
                pass
        print("stored", len(db.all("gemv_int4")), "results in", a.db)


if __name__ == "__main__":
    main()
