"""Multi-GPU test worker: run under torch.distributed.run, one rank per GPU.
    python -m torch.distributed.run --nproc-per-node 2 ... tests/mp_worker.py <scenario> [args]
Exits non-zero on failure; rank 0 prints 'WORKER-OK <scenario>'."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch
import torch.distributed as dist


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-12))


def scenario_allreduce(multimem: bool):
    from mi50grad_b200.parallel.symm import SymmComm
    rank, world = dist.get_rank(), dist.get_world_size()
    comm = SymmComm(part_floats=512 * 5120, use_multimem=multimem)
    dev = comm.device
    for n, twoshot in [(5120, False), (5120, True), (512 * 5120, False), (512 * 5120, True), (40960, None)]:
        for dtype in (torch.float32, torch.float16):
            gens = [torch.Generator().manual_seed(100 + r) for r in range(world)]
            xs = [torch.randn(n, generator=g).to(dtype) for g in gens]
            ref = sum(x.float() for x in xs)
            h0 = torch.randn(n, generator=torch.Generator().manual_seed(7))
            out = h0.to(dev).clone()
            o16 = torch.zeros(n, dtype=torch.float16, device=dev)
            for rep in range(3):                      # epochs advance, parity alternates
                out.copy_(h0)
                comm.all_reduce_into(xs[rank].to(dev), out, residual=True, twoshot=twoshot, out16=o16)
            torch.cuda.synchronize()
            comm.check_status()
            assert _rel(out.cpu(), h0 + ref) < 1e-5, (n, twoshot, dtype)
            assert _rel(o16.cpu(), h0 + ref) < 2e-3
    s = comm.all_reduce_sum(torch.full((64,), float(rank + 1), device=dev))
    assert torch.allclose(s.cpu(), torch.full((64,), world * (world + 1) / 2.0))
    comm.device_barrier()
    torch.cuda.synchronize()
    comm.check_status()
    return comm.has_multimem


def scenario_fused_shapes(multimem: bool):
    """The fused row-parallel projection (INT4 GEMV + exchange over NVLink + residual add + sums of squares
    for the next RMSNorm) at the 27B model's shapes, K = 6144 / tp and 17408 / tp -> 5120, one and five token
    rows, against an fp32 reference: sum over ranks of x_r W_r^T (all-reduced with NCCL) + h.  Both forms
    are checked: the stand-alone GEMV's finisher and the chain kernel's tile-granular exchange."""
    from mi50grad_b200.ops import kernels as K
    from mi50grad_b200.ops import lib as L
    from mi50grad_b200.ops.packing import pack_int4
    from mi50grad_b200.parallel.symm import SymmComm
    from mi50grad_b200.utils.quant import random_int4_linear
    rank, world = dist.get_rank(), dist.get_world_size()
    comm = SymmComm(max_rows=8, hidden=5120, use_multimem=multimem)
    dev, ctx, H = comm.device, comm.ctx(), 5120
    for Kfull in (6144, 17408):
        Kd = Kfull // world
        Kd -= Kd % 64
        gen = torch.Generator().manual_seed(1000 * Kfull + rank)
        lin = random_int4_linear(Kd, H, 128, gen)
        lin.zeros = torch.randint(0, 16, lin.zeros.shape, generator=gen).half()
        pk = pack_int4(lin, dev)
        wd = lin.dense().to(dev)
        for rows in (1, 5):
            x = torch.randn(rows, Kd, generator=gen).half().to(dev)
            h0 = torch.randn(rows, H, generator=torch.Generator().manual_seed(9)).to(dev)
            ref = x.float() @ wd.t()
            dist.all_reduce(ref)
            ref = (ref + h0).cpu()
            # stand-alone GEMV with the finisher
            h = h0.clone()
            ss = K.gemv(pk, x, mode=L.EPI_FINISH, h=h, comm=ctx)
            torch.cuda.synchronize()
            comm.check_status()
            assert _rel(h.cpu(), ref) < 2e-4, ("finisher", Kfull, rows, _rel(h.cpu(), ref))
            assert torch.allclose(ss.sum(-1).cpu(), ref.pow(2).sum(-1), rtol=1e-3)
            # chain kernel, one projection: every 64-column tile is exchanged by the warp that completes it
            h2 = h0.clone()
            ss2 = torch.zeros(rows, H // 64, device=dev)
            op = K.chain_op(pk, x=x, mode=L.EPI_FINISH, h=h2, ss_part=ss2)
            bufs = K.chain_scratch([op], rows, dev)
            for rep in range(3):                      # epochs advance, staging parity alternates
                h2.copy_(h0)
                K.chain([op], rows, bufs, comm=ctx)
            torch.cuda.synchronize()
            comm.check_status()
            assert _rel(h2.cpu(), ref) < 2e-4, ("chain", Kfull, rows, _rel(h2.cpu(), ref))
            assert torch.allclose(ss2.sum(-1).cpu(), ref.pow(2).sum(-1), rtol=1e-3)
            # every rank holds the same bits
            hs = [torch.empty_like(h2) for _ in range(world)]
            dist.all_gather(hs, h2)
            assert all(torch.equal(hs[0], t) for t in hs)
    comm.close()


def scenario_tp_engine(ar_mode: str, multimem: bool, model: str = "tiny"):
    """Small hybrid model at TP=world on GPUs vs the fp32 CPU oracle.  'medium' has 8 query /
    4 KV heads and 8 / 16 DeltaNet heads, so it shards over 8 ranks with every KV head
    replicated on two of them."""
    from mi50grad_b200.config import EngineConfig, tiny_config
    from mi50grad_b200.engine.tp_engine import TPInferenceEngine
    from mi50grad_b200.models.oracle import OracleEngine
    from mi50grad_b200.models.weights import random_model
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = tiny_config() if model == "tiny" else tiny_config(
        hidden_size=512, intermediate_size=2048, num_attention_heads=8, num_key_value_heads=4,
        linear_num_key_heads=8, linear_num_value_heads=16, vocab_size=2048)
    mw = random_model(cfg, 0)
    eng = TPInferenceEngine(cfg, list(range(world)), max_seq_len=128,
                            engine_config=EngineConfig(ar_mode=ar_mode, use_multimem=multimem))
    eng.load_model(mw)
    ids = torch.randint(0, cfg.vocab_size, (16,), generator=torch.Generator().manual_seed(0)).tolist()
    toks = eng.generate_tokens(ids, 8, graph=False)
    toks_g = eng.generate_tokens(ids, 8, graph=True)
    torch.cuda.synchronize()
    eng.check_status()
    assert toks == toks_g, (toks, toks_g)
    if ar_mode == "exact":
        ref, _ = OracleEngine(mw, max_seq_len=128).greedy_generate(ids, 8)
        assert toks == ref, (toks, ref)
    # every rank must have produced the same tokens
    t = torch.tensor(toks, device="cuda")
    ts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(ts, t)
    assert all(torch.equal(ts[0], x) for x in ts)
    lg = eng.compute_logits(None)
    assert lg.shape[0] == cfg.vocab_size
    assert eng.get_allreduce_call_count() > 0
    eng.cleanup()


def scenario_seq_parallel(multimem: bool):
    """Reduce-scatter by token rows + residual + RMSNorm + fp16 all-gather in one kernel: stand-alone at the
    27B prefill shape (and a ragged row count) against an fp32 reference, then the many-row path of the TP
    engine with the sequence-parallel residual stream against the all-reduce placement."""
    from mi50grad_b200.parallel.symm import SymmComm
    rank, world = dist.get_rank(), dist.get_world_size()
    H = 5120
    comm = SymmComm(part_floats=512 * H, hidden=H, use_multimem=multimem)
    dev = comm.device
    for T in (512, 77, 3):
        per = -(-T // world)
        g = torch.Generator().manual_seed(5)
        h0 = torch.randn(T, H, generator=g)
        w = (torch.rand(H, generator=g) + 0.5).half()
        parts = [torch.randn(T, H, generator=torch.Generator().manual_seed(50 + r)) for r in range(world)]
        href = h0 + sum(parts)
        xref = href * torch.rsqrt((href * href).mean(-1, keepdim=True) + 1e-6) * w.float()
        for rep in range(3):                          # epochs advance, parity alternates
            h = h0.to(dev).clone()
            comm.push_rows(parts[rank].to(dev))
            dist.barrier()
            xn = comm.reduce_scatter_norm_allgather(h, w.to(dev), T, 1e-6)
            torch.cuda.synchronize()
            comm.check_status()
            lo, hi = rank * per, min(T, (rank + 1) * per)
            assert _rel(xn.cpu(), xref) < 2e-3, (T, rep, _rel(xn.cpu(), xref))
            if lo < hi:
                assert _rel(h[lo:hi].cpu(), href[lo:hi]) < 1e-5, (T, rep)
            assert _rel(h[T - 1].cpu(), href[T - 1]) < 1e-5, (T, rep)       # the last row lands on every rank
            dist.barrier()
    comm.close()
    # the engine: same tokens and hidden states with either placement
    from mi50grad_b200.config import EngineConfig, tiny_config
    from mi50grad_b200.engine.tp_engine import TPInferenceEngine
    from mi50grad_b200.models.weights import random_model
    cfg = tiny_config(hidden_size=512, intermediate_size=2048, num_attention_heads=8, num_key_value_heads=4,
                      linear_num_key_heads=8, linear_num_value_heads=16, vocab_size=2048)
    mw = random_model(cfg, 0)
    ids = torch.randint(0, cfg.vocab_size, (70,), generator=torch.Generator().manual_seed(0)).tolist()
    outs = []
    for sp in (1, 0):
        eng = TPInferenceEngine(cfg, list(range(world)), max_seq_len=128,
                                engine_config=EngineConfig(use_multimem=multimem, seq_parallel=sp))
        eng.load_model(mw)
        toks = eng.generate_tokens(ids, 6, graph=False)
        assert bool(eng.engine.seq_parallel) == bool(sp)
        eng.engine.reset()
        first = eng.engine.prefill_tokens_tc(ids)
        xn_last = eng.engine.buf["p_xn"][len(ids) - 1].float().cpu().clone()
        h_last = eng.engine.buf["h"][0].float().cpu().clone()
        torch.cuda.synchronize()
        eng.check_status()
        outs.append((toks, first, xn_last, h_last))
        eng.cleanup()
    assert outs[0][0] == outs[1][0] and outs[0][1] == outs[1][1], (outs[0][0], outs[1][0])
    assert _rel(outs[0][2], outs[1][2]) < 5e-3 and _rel(outs[0][3], outs[1][3]) < 1e-3


def scenario_spec():
    """Speculative verification and many-row steps at TP=world against the oracle: a draft tree
    (GEMV path), three sequences with chains (tensor-core path), batched decode of 10 sequences."""
    from mi50grad_b200.config import EngineConfig, tiny_config
    from mi50grad_b200.engine.tp_engine import TPInferenceEngine
    from mi50grad_b200.models.oracle import OracleEngine
    from mi50grad_b200.models.weights import random_model
    world = dist.get_world_size()
    cfg = tiny_config()
    mw = random_model(cfg, 5)
    eng = TPInferenceEngine(cfg, list(range(world)), max_seq_len=128, max_batch=10, engine_config=EngineConfig())
    eng.load_model(mw)
    orc = OracleEngine(mw, max_seq_len=128, max_batch=10)
    prm = lambda n, s: torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(s)).tolist()
    wrong = lambda t: (t + 3) % cfg.vocab_size
    prompts = [prm(6 + i, 40 + i) for i in range(10)]
    refs = [orc.greedy_generate(p, 9, seq=i)[0] for i, p in enumerate(prompts)]
    for i, p in enumerate(prompts):
        assert eng.prefill_tokens(p, seq=i) == refs[i][0], i
    # tree on sequence 0 (5 drafts + pending token = 6 rows)
    r = refs[0]
    drafts, parents = [wrong(r[1]), r[1], r[2], wrong(r[2]), wrong(r[3])], [-1, -1, 1, 1, 2]
    (acc, nxt), = eng.spec_step([drafts], [parents], [0])
    assert acc == [r[1], r[2]] and nxt == r[3], (acc, nxt, r[:5])
    # chains on sequences 1..3 (12 rows: tensor-core path)
    dr, pa, exp = [], [], []
    for i in (1, 2, 3):
        r = refs[i]
        n_ok = i - 1
        d = [r[1 + k] if k < n_ok else wrong(r[1 + k]) for k in range(3)]
        dr.append(d); pa.append([-1, 0, 1]); exp.append((d[:n_ok], r[1 + n_ok]))
    res = eng.spec_step(dr, pa, [1, 2, 3])
    assert [(a, n) for a, n in res] == exp, (res, exp)
    # batched decode of the untouched sequences 4..9 plus the advanced ones: all ten
    out = eng.decode_tokens(2, seqs=list(range(10)), graph=False).cpu()
    adv = {0: 3, 1: 1, 2: 2, 3: 3}
    for i in range(10):
        a = adv.get(i, 0)
        assert out[:, i].tolist() == refs[i][a + 1:a + 3], (i, out[:, i].tolist(), refs[i])
    torch.cuda.synchronize()
    eng.check_status()
    eng.cleanup()


def scenario_wait_timeout():
    """A flag that nobody raises: the bounded wait must return with a status and
    leave the context usable.  Plain peer loads, no multicast."""
    from mi50grad_b200.parallel.comm import CommTimeout
    from mi50grad_b200.parallel.symm import SymmComm
    comm = SymmComm(use_multimem=False, wait_us=200_000)
    dev = comm.device
    x = torch.ones(4096, device=dev)
    out = torch.zeros(4096, device=dev)
    comm.all_reduce_into(x, out, withhold_signal=True)      # every rank withholds: all time out
    torch.cuda.synchronize()
    try:
        comm.check_status()
    except CommTimeout as e:
        msg = str(e)
    else:
        raise AssertionError("expected CommTimeout")
    assert "all-reduce" in msg
    # the context is still usable, and after a host-side re-synchronisation so is the communicator
    y = (torch.ones(8, device=dev) * 2).sum().item()
    assert y == 16
    dist.barrier()
    comm2 = SymmComm(use_multimem=False)
    comm2.all_reduce_into(x, out)
    torch.cuda.synchronize()
    comm2.check_status()
    assert float(out[0]) == dist.get_world_size()


def scenario_failure_detection():
    """Failure detection and recovery wired into the tensor-parallel engine, with no GPU fault anywhere:
    (1) recover() -- a new symmetric-memory communicator, a rebuilt driver, sequences restored from
    snapshots -- continues with exactly the tokens of the uninterrupted run; (2) a rank that leaves between
    steps (nothing of its in flight) is seen by the other rank before its next launch."""
    import time
    from mi50grad_b200.config import EngineConfig, tiny_config
    from mi50grad_b200.engine.tp_engine import TPInferenceEngine
    from mi50grad_b200.models.weights import random_model
    from mi50grad_b200.utils.watchdog import RankFailure
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = tiny_config()
    eng = TPInferenceEngine(cfg, list(range(world)), max_seq_len=128,
                            engine_config=EngineConfig(use_multimem=False, wait_budget_us=500_000))
    eng.load_model(random_model(cfg, 0))
    eng.enable_failure_detection(heartbeat_s=0.05, timeout_s=3.0)
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(2)).tolist()
    eng.generate_tokens(ids, 4, graph=False)
    snaps = eng.snapshot_all([0])
    a = eng.decode_tokens(3, graph=False).cpu().tolist()
    old = eng.comm
    eng.recover(snaps)
    assert eng.comm is not old
    b = eng.decode_tokens(3, graph=False).cpu().tolist()
    torch.cuda.synchronize()
    eng.check_status()
    assert a == b, (a, b)
    dist.barrier()
    if rank == world - 1:
        eng._heartbeat.mark_failed("leaving between steps")      # this rank issues nothing from here on
    else:
        t0, seen = time.time(), None
        while time.time() - t0 < 10 and seen is None:
            try:
                eng._before_step()
                time.sleep(0.02)
            except RankFailure as e:
                seen = e
        assert seen is not None and seen.rank == world - 1 and "leaving" in seen.reason
        with pytest_raises(RankFailure):
            eng.decode_tokens(1, graph=False)                     # refused on the host: no kernel is launched
    eng.cleanup()


class pytest_raises:
    def __init__(self, exc):
        self.exc = exc

    def __enter__(self):
        return self

    def __exit__(self, t, v, tb):
        assert t is not None and issubclass(t, self.exc), f"expected {self.exc.__name__}"
        return True


def scenario_sample():
    """Non-greedy generation under TP: every rank samples from its own vocabulary slice and the ranks
    exchange candidate lists inside the sampling kernel; the ranks agree, and both the kept candidates and
    the draw equal the one-rank sampler run on the gathered logits."""
    from mi50grad_b200.config import EngineConfig, tiny_config
    from mi50grad_b200.engine.tp_engine import TPInferenceEngine
    from mi50grad_b200.generate.generate import TextGenerator
    from mi50grad_b200.generate.sampler import SamplingParams
    from mi50grad_b200.models.weights import random_model
    from mi50grad_b200.ops import kernels as K
    world = dist.get_world_size()
    cfg = tiny_config()
    eng = TPInferenceEngine(cfg, list(range(world)), max_seq_len=128, engine_config=EngineConfig())
    eng.load_model(random_model(cfg, 5))
    gen = TextGenerator(eng)
    prompt = [3, 14, 15, 92, 65]
    sp = SamplingParams(temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.1, max_tokens=12, seed=11)
    ids = gen.generate_ids(prompt, sp)
    assert len(ids) == 12 and all(0 <= t < cfg.vocab_size for t in ids)
    again = gen.generate_ids(prompt, sp)
    assert again == ids                                            # same seed, same stream
    other = gen.generate_ids(prompt, SamplingParams(temperature=0.8, top_k=40, top_p=0.9, max_tokens=12, seed=12))
    t = torch.tensor(ids + other, device="cuda")
    all_t = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(all_t, t)
    assert all(torch.equal(a, t) for a in all_t)                   # every rank drew the same tokens
    # the gathered logits are the full vocabulary: a near-zero temperature draw is their arg-max
    full = eng.compute_logits(None)
    assert full.numel() == cfg.vocab_size
    cold = K.sample_top_p(full.reshape(1, -1).clone(), 1e-4, 1, 1.0, seed=1)
    assert int(cold[0]) == int(full.argmax())
    first = gen.prefill(prompt)
    assert first == int(eng.compute_logits(None).argmax())         # gathered logits of the last step
    # slice-local sampler == one-rank sampler on the gathered logits, for three parameter sets
    core = eng.engine
    past = torch.tensor([sorted(set(prompt + ids))], dtype=torch.int32, device="cuda")
    npast = torch.tensor([past.shape[1]], dtype=torch.int32, device="cuda")
    for temp, tk, tpp, pen in ((0.8, 40, 0.9, 1.1), (1.3, 0, 0.95, 1.0), (0.5, 7, 1.0, 1.4)):
        full = eng.compute_logits(None).reshape(1, -1).clone()
        ref_tok, ref_ids, ref_p = K.sample_top_p(full, temp, tk, tpp, pen, past, npast, seed=77, debug=True)
        local = core.logits(1).clone()
        tok, got_ids, got_p = K.sample_top_p(local, temp, tk, tpp, pen, past, npast, seed=77, debug=True,
                                             vocab_offset=core.spec.vocab[0], comm=core._comm_ctx(),
                                             vocab_total=cfg.vocab_size)
        torch.cuda.synchronize()
        eng.check_status()
        assert int(tok[0]) == int(ref_tok[0]), (temp, tk, tpp, pen)
        assert torch.equal(got_ids, ref_ids)
        assert torch.allclose(got_p, ref_p, atol=1e-6)
    eng.cleanup()


def main():
    scenario = sys.argv[1]
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    try:
        if scenario == "allreduce":
            mm = scenario_allreduce(sys.argv[2] == "multimem")
            extra = f"multimem={mm}"
        elif scenario == "tp_engine":
            scenario_tp_engine(sys.argv[2], sys.argv[3] == "multimem", sys.argv[4] if len(sys.argv) > 4 else "tiny")
            extra = sys.argv[2]
        elif scenario == "fused_shapes":
            scenario_fused_shapes(sys.argv[2] == "multimem")
            extra = sys.argv[2]
        elif scenario == "spec":
            scenario_spec()
            extra = ""
        elif scenario == "seq_parallel":
            scenario_seq_parallel(sys.argv[2] == "multimem")
            extra = sys.argv[2]
        elif scenario == "sample":
            scenario_sample()
            extra = ""
        elif scenario == "failure_detection":
            scenario_failure_detection()
            extra = ""
        elif scenario == "wait_timeout":
            scenario_wait_timeout()
            extra = ""
        else:
            raise SystemExit(f"unknown scenario {scenario}")
        dist.barrier()
        if dist.get_rank() == 0:
            print(f"WORKER-OK {scenario} {extra}", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
