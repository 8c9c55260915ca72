"""Metrics, guard bands, heartbeat/watchdog and recovery -- everything on the host (CPU, gloo)."""
import json

import pytest
import torch
import torch.distributed as dist

from helpers import free_port, run_gloo
from mi50grad_b200.config import tiny_config
from mi50grad_b200.models.oracle import OracleEngine
from mi50grad_b200.models.weights import random_model
from mi50grad_b200.parallel.comm import TorchDistComm
from mi50grad_b200.parallel.sharding import shard_model
from mi50grad_b200.utils.guards import GuardedAllocator, GuardError
from mi50grad_b200.utils.metrics import Metrics, PhaseTimer
from mi50grad_b200.utils.watchdog import DictStore, Heartbeat, RankFailure, Watchdog, recover


def test_metrics_record_and_phase_timer(tmp_path):
    m = Metrics(run="t", n_gpus=2, tokens=256, steps=128, seconds=0.64, drafted=40, accepted=22)
    m.finish()
    assert abs(m.ms_per_step - 5.0) < 1e-9 and abs(m.tok_per_s - 400.0) < 1e-9
    d = json.loads(m.to_json())
    assert d["acceptance_rate"] == 0.55 and d["n_gpus"] == 2
    m.dump(str(tmp_path / "m.jsonl"))
    assert json.loads((tmp_path / "m.jsonl").read_text().strip())["tokens"] == 256
    t = PhaseTimer(use_cuda=False)
    with t.phase("a"):
        sum(range(1000))
    with t.phase("a"):
        pass
    assert t.summary()["a"] >= 0.0


def test_guard_bands_detect_out_of_bounds_writes():
    g = GuardedAllocator("cpu", band_bytes=256)
    x = g.zeros("scratch", (4, 8), torch.float32)
    y = g.zeros("counters", 10, torch.int32)
    x.fill_(1.0); y.fill_(7)
    g.check_all()                                              # writes inside are fine
    raw, nbytes = g._bufs["scratch"]
    raw[g.band + nbytes + 3] = 0                               # one byte past the end
    with pytest.raises(GuardError) as e:
        g.check_all()
    assert "scratch" in str(e.value) and str(nbytes + 3) in str(e.value)
    raw[g.band + nbytes + 3] = 0xA5
    raw2, _ = g._bufs["counters"]
    raw2[g.band - 1] = 1                                       # one byte before the start
    assert g.check("counters") == [-1]


def test_watchdog_detects_silent_failed_and_stuck_ranks():
    now = [100.0]
    clock = lambda: now[0]
    store = DictStore()
    hbs = [Heartbeat(store, r, clock=clock) for r in range(3)]
    wd = Watchdog(store, 0, 3, timeout_s=2.0, clock=clock)
    with pytest.raises(RankFailure) as e:
        wd.check()
    assert e.value.rank == 1 and "no heartbeat" in e.value.reason
    for h in hbs:
        h.beat(5)
    wd.check()
    now[0] += 1.5
    hbs[1].beat(6)
    wd.check()                                                 # rank 2 is 1.5 s old: within the timeout
    now[0] += 1.0
    hbs[1].beat(7)
    with pytest.raises(RankFailure) as e:
        wd.check()
    assert e.value.rank == 2 and "old" in e.value.reason
    hbs[2].beat(7)
    hbs[1].mark_failed("CommTimeout in all-reduce")
    with pytest.raises(RankFailure) as e:
        wd.check()
    assert e.value.rank == 1 and "CommTimeout" in e.value.reason


def _fail_and_recover(rank, world, port2, fail_step, n_steps):
    """TP=2 decode; rank 1 fails between steps (an exception on the host, nothing in flight); both
    ranks learn of it through the store, re-bootstrap a new process group and continue from the
    snapshot taken before the failed step."""
    cfg = tiny_config()
    mw = shard_model(random_model(cfg, 0), world, rank)
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, prefix="hb0")
    wd = Watchdog(store, rank, world, timeout_s=20.0, prefix="hb0")
    eng = OracleEngine(mw, world, rank, TorchDistComm())
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(0)).tolist()
    h = eng.prefill_step(eng.embed(ids))
    toks, detected = [], None
    step = 0
    while len(toks) < n_steps:
        snap = (eng.snapshot(0), h.clone(), list(toks))
        try:
            if rank == 1 and step == fail_step and detected is None:
                raise RuntimeError("injected host failure")
            hb.beat(step)                                      # announce: about to enter the collectives of `step`
            wd.wait_for_step(step)                             # every peer announced it too (or is known to have failed)
            t = int(torch.argmax(eng.compute_logits(h)))
            h = eng.decode_step(eng.embed([t])[0])
            toks.append(t)
            step += 1
        except (RuntimeError, RankFailure) as e:
            if detected is not None:
                raise
            detected = str(e)
            if not isinstance(e, RankFailure):
                hb.mark_failed(detected)
            # recovery: new process group on a fresh rendezvous, state back to the last snapshot
            def rebootstrap():
                dist.destroy_process_group()
                dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port2}", rank=rank, world_size=world)
                return TorchDistComm()
            def restore(s):
                eng.restore(s[0], 0)
            eng.comm = recover(rebootstrap, restore, [snap])
            h, toks = snap[1], snap[2]
            store = dist.distributed_c10d._get_default_store()
            hb = Heartbeat(store, rank, prefix="hb1")
            wd = Watchdog(store, rank, world, timeout_s=20.0, prefix="hb1")
    return toks, detected


def test_run_guarded_recovers_once_and_clears_failure_marks():
    """The retry wrapper around engine steps: a CommTimeout (or a peer's failure mark) triggers exactly one
    recover() from the snapshots, after which the step is tried again; a mark that was withdrawn no longer
    stops the peers."""
    from mi50grad_b200.parallel.comm import CommTimeout
    from mi50grad_b200.utils.watchdog import DictStore, Heartbeat, RankFailure, Watchdog, run_guarded

    class FakeEngine:
        def __init__(self):
            self.recovered, self.calls = [], 0

        def synchronize(self):
            pass

        def check_status(self):
            pass

        def recover(self, snaps):
            self.recovered.append(list(snaps))

    eng = FakeEngine()

    def step():
        eng.calls += 1
        if eng.calls == 1:
            raise CommTimeout("rank 0: bounded wait expired")
        return "tokens"
    assert run_guarded(eng, step, ["snap0"], retries=1) == "tokens"
    assert eng.recovered == [["snap0"]] and eng.calls == 2
    eng2 = FakeEngine()
    with pytest.raises(CommTimeout):
        run_guarded(eng2, lambda: (_ for _ in ()).throw(CommTimeout("again")), [], retries=1)
    assert len(eng2.recovered) == 1
    store = DictStore()
    hb0, hb1 = Heartbeat(store, 0), Heartbeat(store, 1)
    hb0.beat(); hb1.beat()
    wd = Watchdog(store, 0, 2, timeout_s=60)
    hb1.mark_failed("exchange timed out")
    with pytest.raises(RankFailure):
        wd.check()
    hb1.clear_failed()
    wd.check()


def test_rank_failure_is_detected_and_run_recovers():
    cfg = tiny_config()
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(0)).tolist()
    ref, _ = OracleEngine(random_model(cfg, 0)).greedy_generate(ids, 6)
    res = run_gloo(_fail_and_recover, 2, free_port(), 3, 6)
    for toks, detected in res:
        assert toks == ref
    assert "injected" in res[1][1]
    assert "reported failure" in res[0][1] and "injected" in res[0][1]


def test_activation_quant_per_row_matches_per_tensor_on_one_row():
    import torch
    from mi50grad_b200.utils import quant as Q
    x = torch.randn(1, 256)
    q1, s1 = Q.quantize_activation_int8(x)
    q2, s2 = Q.quantize_activation_int8(x, per_row=True)
    assert torch.equal(q1, q2) and torch.allclose(s1, s2[0])
    x = torch.randn(3, 64) * torch.tensor([[1.0], [10.0], [0.1]])
    q, s = Q.quantize_activation_int8(x, per_row=True)
    assert s.shape == (3,) and q.abs().amax(dim=1).tolist() == [127, 127, 127]
    assert torch.allclose(q.float() * s[:, None], x, atol=float(s.max()) * 0.51)
