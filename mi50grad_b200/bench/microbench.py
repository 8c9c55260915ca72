"""Kernel micro-benchmarks with roofline fractions.

    python -m mi50grad_b200.bench.microbench gemv [--tp 1] [--rows 1] [--iters 20]

Each shape is timed with CUDA events over `iters` launches that rotate through
enough independent weight copies to exceed the 126 MB L2, after 3 warm-ups;
achieved bandwidth is weight bytes / time and the fraction is taken against the
measured copy bandwidth in MEASURED_PEAKS.json (fallback 6.65 TB/s).
(reference counterparts: bench/micro/*.hip.cpp, tests/bench_*.py)
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def measured_peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                     "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


def time_launches(fn, n_variants: int, iters: int, warmup: int = 3) -> float:
    """Mean microseconds per launch of fn(i % n_variants)."""
    for i in range(warmup):
        fn(i % n_variants)
    torch.cuda.synchronize()
    # the launches are captured in a CUDA graph so that host launch cost is not what is timed
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i % n_variants)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def bench_gemv(tp: int, rows: int, iters: int, only=None):
    from ..config import qwen35_27b
    from ..ops import kernels as K
    from ..ops import lib as L
    from ..ops.packing import random_packed_int4
    cfg = qwen35_27b()
    H, F = cfg.hidden_size, cfg.intermediate_size // tp
    qd, kvd = cfg.full_attn_q_dim // tp, max(cfg.head_dim, cfg.full_attn_kv_dim // tp)
    shapes = {
        "ffn_gate_up(silu)": (H, 2 * F, L.EPI_SILU_PAIR),
        "ffn_down(finish)": (F, H, L.EPI_FINISH),
        "attn_qkv": (H, 2 * qd + 2 * kvd, L.EPI_STORE_F16),
        "deltanet_in_proj": (H, (2 * cfg.linear_attn_key_dim + 2 * cfg.linear_attn_value_dim) // tp, L.EPI_STORE_F16),
        "attn_o_proj(finish)": (qd, H, L.EPI_FINISH),
    }
    hbm, _, src = measured_peaks()
    dev = torch.device("cuda")
    out = []
    for name, (Kd, N, mode) in shapes.items():
        if only and only not in name:
            continue
        one = random_packed_int4(Kd, N, 128, dev)
        nvar = max(2, int(300e6 // one.nbytes()) + 1)
        pks = [one] + [random_packed_int4(Kd, N, 128, dev) for _ in range(nvar - 1)]
        x = torch.randn(rows, Kd, device=dev).half()
        o16 = torch.zeros(rows, one.n_pad, dtype=torch.float16, device=dev)
        h = torch.zeros(rows, N, device=dev)
        xn = torch.zeros(rows, N, dtype=torch.float16, device=dev)
        lp = torch.zeros(rows, N, device=dev)
        w = torch.ones(N, dtype=torch.float16, device=dev)
        scratch = torch.empty(max(1, one.k_splits * rows * one.n_pad), device=dev)
        counters = torch.zeros(one.n_pad // 128 + 2, dtype=torch.int32, device=dev)

        def run(i):
            if mode == L.EPI_FINISH:
                K.gemv(pks[i], x, mode=mode, fin_flags=L.FIN_NO_COMM, h=h, norm_w=w,
                       scratch=scratch, counters=counters)
            else:
                K.gemv(pks[i], x, out=o16, mode=mode, scratch=scratch, counters=counters)
        us = time_launches(run, nvar, iters)
        gbs = one.nbytes() / us / 1e3
        out.append({"kernel": "gemv_int4", "shape": name, "K": Kd, "N": N, "rows": rows, "tp": tp,
                    "grid": [one.n_pad // 128, one.k_splits], "L": one.L, "us": round(us, 2),
                    "weight_mb": round(one.nbytes() / 1e6, 2), "gb_s": round(gbs, 1),
                    "frac_of_hbm": round(gbs / hbm, 3), "peak_source": src})
        print(json.dumps(out[-1]), flush=True)
    return out


def bench_fused(iters: int):
    """The fused row-parallel projection: INT4 GEMV + all-reduce + residual add (+ lazy RMSNorm sums) as ONE
    kernel at TP = world size, and stand-alone all-reduces of 10 KB / 5 MB, each against NCCL
    all-reduce plus separate kernels.  Run under torch.distributed.run; times are max over ranks."""
    import torch.distributed as dist
    from ..config import qwen35_27b
    from ..ops import kernels as K
    from ..ops import lib as L
    from ..ops.packing import random_packed_int4
    from ..parallel.symm import SymmComm
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    tp, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", local)
    cfg = qwen35_27b()
    H = cfg.hidden_size
    hbm, _, src = measured_peaks()
    results = []

    def mx(us):
        t = torch.tensor([us], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for multimem in (True, False):
        comm = SymmComm(part_floats=512 * H, use_multimem=multimem)
        ctx = comm.ctx()
        for name, Kfull in (("o_proj", cfg.full_attn_q_dim), ("down_proj", cfg.intermediate_size)):
            Kd = Kfull // tp
            nvar = 8
            pks = [random_packed_int4(Kd, H, 128, dev) for _ in range(nvar)]
            x = torch.randn(1, Kd, device=dev).half()
            h = torch.zeros(1, H, device=dev)
            ss = torch.zeros(1, H // 128, device=dev)
            scratch = torch.empty(max(1, pks[0].k_splits * pks[0].n_pad), device=dev)
            counters = torch.zeros(pks[0].n_pad // 128 + 2, dtype=torch.int32, device=dev)
            part = torch.zeros(1, H, device=dev)

            def fused(i):
                K.gemv(pks[i], x, mode=L.EPI_FINISH, h=h, ss_part=ss, comm=ctx, scratch=scratch, counters=counters)

            cops = [K.chain_op(pk, x=x, mode=L.EPI_FINISH, h=h, ss_part=torch.zeros(1, H // 64, device=dev)) for pk in pks]
            cbufs = K.chain_scratch(cops, 1, dev)

            def fused_chain(i):
                K.chain([cops[i]], 1, cbufs, comm=ctx)

            def unfused(i):
                K.gemv(pks[i], x, out=part, mode=L.EPI_STORE_F32, scratch=scratch, counters=counters)
                dist.all_reduce(part)
                K.add_rmsnorm(h, torch.ones(H, dtype=torch.float16, device=dev), part)
            dist.barrier()
            us_f = mx(time_launches(fused, nvar, iters))
            dist.barrier()
            us_c = mx(time_launches(fused_chain, nvar, iters))
            dist.barrier()
            us_u = mx(time_launches(unfused, nvar, iters))
            comm.check_status()
            # in-kernel time stamps of one finisher launch (globaltimer, relative to the kernel's start)
            comm.trace_enabled = True
            K.gemv(pks[0], x, mode=L.EPI_FINISH, h=h, ss_part=ss, comm=comm.ctx(), scratch=scratch, counters=counters)
            torch.cuda.synchronize()
            trace = comm.last_exchange_trace()
            comm.trace_enabled = False
            # roofline: the slower of streaming this rank's weight shard from HBM and moving the
            # partial vectors over NVLink (20 KB per peer, latency bound: reported for context)
            t_hbm = pks[0].nbytes() / (hbm * 1e3)
            results.append({"kernel": "int4_gemv_ar_residual", "shape": name, "K_local": Kd, "N": H, "tp": tp,
                            "multimem": comm.has_multimem, "fused_us": round(us_f, 2),
                            "chain_tile_exchange_us": round(us_c, 2),
                            "gemv+nccl+add_us": round(us_u, 2), "speedup": round(us_u / us_f, 2),
                            "hbm_floor_us": round(t_hbm, 2), "frac_of_roofline": round(t_hbm / us_f, 3),
                            "finisher_trace_ns": trace, "peak_source": src})
            if rank == 0:
                print(json.dumps(results[-1]), flush=True)
        for n, label in ((H, "10KB fp16 payload (5120 elems)"), (512 * H, "5MB fp16 payload (512x5120)")):
            src_t = torch.randn(n, device=dev).half()
            out = torch.zeros(n, device=dev)
            for twoshot in (False, True):
                def ours(i):
                    comm.all_reduce_into(src_t, out, residual=True, twoshot=twoshot)
                dist.barrier()
                us = mx(time_launches(ours, 1, iters))
                comm.check_status()
                results.append({"kernel": "allreduce_residual", "payload": label, "tp": tp,
                                "algo": "two-shot" if twoshot else "one-shot", "multimem": comm.has_multimem,
                                "us": round(us, 2)})
                if rank == 0:
                    print(json.dumps(results[-1]), flush=True)
            if multimem:
                buf = torch.randn(n, device=dev).half()
                acc = torch.zeros(n, device=dev)

                def nccl(i):
                    dist.all_reduce(buf)
                    K.residual_add_(acc, buf)
                dist.barrier()
                us = mx(time_launches(nccl, 1, iters))
                results.append({"kernel": "nccl_allreduce+residual_add", "payload": label, "tp": tp, "us": round(us, 2)})
                if rank == 0:
                    print(json.dumps(results[-1]), flush=True)
        comm.close()
    dist.barrier()
    dist.destroy_process_group()
    return results


def bench_nvlink(iters: int):
    """NVLink probes (reference: src/kernels/p2p_bandwidth_kernels.hip:187-278 and
    bench/PCIe4_BANDWIDTH_REPORT.md): read bandwidth from local memory, from a peer's memory with plain
    loads, through the multicast address with multimem.ld_reduce (payload counted once), write bandwidth
    into a peer's memory, for 10 KB ... 64 MB; and the latency of dependent loads, local and peer.
    Run under torch.distributed.run with >= 2 ranks; every figure is the slowest rank's."""
    import torch.distributed as dist
    from ..ops import kernels as K
    from ..parallel.symm import SymmComm
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    tp, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", local)
    comm = SymmComm(part_floats=8 * 1024 * 1024, use_multimem=True)          # 64 MB staging region per rank
    peer = (rank + 1) % tp
    me_ptr, peer_ptr = comm.peer_ptrs[rank], comm.peer_ptrs[peer]
    sink = torch.empty(64 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def mx(v):
        t = torch.tensor([v], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    res = []
    for nbytes in (10 * 1024, 160 * 1024, 1024 * 1024, 8 * 1024 * 1024, 64 * 1024 * 1024):
        ctas = max(1, min(296, nbytes // (16 * 512)))
        cases = {"local_read": lambda: K.probe_read(me_ptr, nbytes, ctas=ctas),
                 "peer_read": lambda: K.probe_read(peer_ptr, nbytes, ctas=ctas),
                 "peer_write": lambda: K.probe_read(sink.data_ptr(), nbytes, dst_ptr=peer_ptr, ctas=ctas)}
        if comm.has_multimem:
            cases["multimem_ld_reduce"] = lambda: K.probe_read(comm.multicast_ptr, nbytes, multimem=True, ctas=ctas)
        row = {"probe": "bandwidth", "bytes": nbytes, "tp": tp, "ctas": ctas}
        for name, fn in cases.items():
            dist.barrier()
            us = mx(time_launches(lambda i: fn(), 1, iters))
            row[name + "_us"] = round(us, 2)
            row[name + "_gb_s"] = round(nbytes / us / 1e3, 1)
        res.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    # dependent-load latency: a chain of indices with a 4 KB stride, walked from local and from peer memory
    n = 1 << 16
    chain = ((torch.arange(n, dtype=torch.int64) + 1024) % n).to(torch.int32)
    region = torch.empty(0)
    local_view = comm.buf[: n * 4].view(torch.int32)
    local_view.copy_(chain.to(dev))
    torch.cuda.synchronize()
    dist.barrier()
    lat = {"probe": "latency", "tp": tp, "hops": 2000,
           "local_ns": round(mx(K.probe_latency(local_view, 2000)), 1),
           "peer_ns": round(mx(K.probe_latency(local_view, 2000, chain_ptr=peer_ptr)), 1)}
    res.append(lat)
    if rank == 0:
        print(json.dumps(lat), flush=True)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return res


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemv", "fused", "nvlink"])
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default=None)
    a = ap.parse_args(argv)
    if a.what == "gemv":
        bench_gemv(a.tp, a.rows, a.iters, a.only)
    elif a.what == "nvlink":
        bench_nvlink(a.iters)
    else:
        bench_fused(a.iters)


if __name__ == "__main__":
    main()
