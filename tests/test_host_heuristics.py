"""Host-side choices that shape the GPU launches: the GEMV launch shape and the engine switches."""
import os

from mi50grad_b200.config import EngineConfig
from mi50grad_b200.ops.packing import GEMV_WK, launch_shape


def test_launch_shape_fills_one_wave_and_covers_k():
    for K, N in [(5120, 34816), (5120, 16384), (5120, 14336), (17408, 5120), (6144, 5120), (768, 5120), (2176, 5120),
                 (1536, 5120), (4352, 5120), (5120, 2048), (5120, 4352)]:
        KB, NTL = -(-K // 64), -(-N // 128) * 8
        ks, L = launch_shape(KB, NTL, 1)
        assert ks >= 1 and L >= 1
        assert ks * L * GEMV_WK >= KB                      # every k-block has an owner
        assert (ks - 1) * L * GEMV_WK < KB                 # no empty split
        assert (NTL * 16 // 128) * ks <= 2 * 148 or ks == 1   # two resident CTAs per SM, one wave
        # activation staging of one CTA stays inside its shared-memory share
        assert 2 * GEMV_WK * L * 2 * 64 <= 32_000


def test_launch_shape_short_k_is_not_split():
    # a row-parallel shard under 8-way tensor parallelism: the cross-CTA round trip costs more than it spreads
    for K in (768, 1024, 1536):
        ks, _ = launch_shape(-(-K // 64), 5120 // 16, 1)
        assert ks == 1


def test_launch_shape_more_rows_need_more_splits_or_shorter_slices():
    KB, NTL = 17408 // 64, 5120 // 16
    ks1, L1 = launch_shape(KB, NTL, 1)
    ks8, L8 = launch_shape(KB, NTL, 8)
    assert 2 * GEMV_WK * L8 * 9 * 64 <= 32_000
    assert ks8 >= ks1 and L8 <= L1


def test_engine_switch_defaults_and_environment(monkeypatch):
    for k in ("B200GRAD_CHAIN", "B200GRAD_SEQ_PARALLEL", "B200GRAD_AR_MODE", "B200GRAD_GRAPH", "B200GRAD_MULTIMEM"):
        monkeypatch.delenv(k, raising=False)
    e = EngineConfig()
    assert e.use_chain == -1 and e.seq_parallel == 1 and e.ar_mode == "exact" and e.use_graph and e.use_multimem
    monkeypatch.setenv("B200GRAD_CHAIN", "0")
    monkeypatch.setenv("B200GRAD_SEQ_PARALLEL", "0")
    e = EngineConfig()
    assert e.use_chain == 0 and e.seq_parallel == 0
    monkeypatch.setenv("B200GRAD_AR_MODE", "deferred_consistent")
    monkeypatch.setenv("B200GRAD_MULTIMEM", "0")
    e = EngineConfig.from_env()
    assert e.ar_mode == "deferred_consistent" and not e.use_multimem
    assert e.replace(use_chain=1).use_chain == 1 and e.use_chain == 0
