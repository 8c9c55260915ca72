"""Small, self-contained workloads for profiler captures and kernel timing.

    python -m mi50grad_b200.bench.profile_cases <case> [--time]

Each case launches one kernel family a few times on inputs larger than L2 but
only a few hundred MB in total, brackets the launches of interest with
cudaProfilerStart/Stop, and with --time prints CUDA-event timings taken from a
graph replay instead.  Capture one case and one kernel at a time, after the same
command has exited 0 without a profiler, and never let the profiler touch the
clocks of a shared GPU:

    ncu --clock-control none --profile-from-start off -k regex:<kernel> -c 3 \
        python -m mi50grad_b200.bench.profile_cases <case>

cases: gemv_gateup, gemv_down, gemm_int4, gemm_dense, attn_decode, attn_rows, attn_prefill,
       deltanet_step, deltanet_chunk, spec_step, prefill, decode_step, linear_q8
"""
from __future__ import annotations

import argparse

import torch

from ..ops import kernels as K
from ..ops import lib as L
from ..ops.packing import random_packed_int4
from .microbench import time_launches


def _profiled(fn, reps: int = 2):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()


def _report(name, us, bytes_=0.0, flops=0.0):
    msg = f"{name}: {us:.1f} us"
    if bytes_:
        msg += f"  {bytes_ / us / 1e3:.0f} GB/s"
    if flops:
        msg += f"  {flops / us / 1e6:.0f} TFLOP/s"
    print(msg, flush=True)


def case_gemv(which: str, timed: bool):
    dev = torch.device("cuda")
    Kd, N, mode = (5120, 34816, L.EPI_SILU_PAIR) if which == "gemv_gateup" else (17408, 5120, L.EPI_STORE_F32)
    pks = [random_packed_int4(Kd, N, 128, dev) for _ in range(3)]          # rotate: 3 x 89 MB > L2
    x = torch.randn(1, Kd, device=dev).half()
    out = torch.zeros(1, N, dtype=torch.float16 if mode == L.EPI_SILU_PAIR else torch.float32, device=dev)
    scratch = torch.zeros(8 * 1024 * 1024, dtype=torch.float32, device=dev)
    counters = torch.zeros(8192, dtype=torch.int32, device=dev)
    from ..engine.engine import DeviceLinear
    lins = [DeviceLinear(packed=p) for p in pks]
    run = lambda i=0: K.gemv(lins[i % 3], x, out=out, mode=mode, scratch=scratch, counters=counters)
    if timed:
        _report(which, time_launches(run, 3, 12), bytes_=pks[0].nbytes())
    else:
        state = {"i": 0}
        def step():
            run(state["i"]); state["i"] += 1
        _profiled(step, 3)


def case_gemm(which: str, timed: bool):
    dev = torch.device("cuda")
    if which == "gemm_int4":
        # (K, N, T, tokens per CTA, 128-output halves per CTA, CTA pairs)
        shapes = [(17408, 5120, 512, 176, 1, 0), (5120, 34816, 512, 512, 1, 0), (5120, 34816, 80, 80, 1, 0),
                  (5120, 34816, 512, 512, 1, 1)]
        if timed:
            shapes += [(5120, 34816, 512, 256, 1, 1), (5120, 34816, 512, 256, 2, 0),
                       (5120, 16384, 512, 512, 1, 0), (5120, 16384, 512, 512, 1, 1), (5120, 16384, 512, 256, 1, 1),
                       (5120, 16384, 512, 256, 2, 0), (17408, 5120, 512, 512, 1, 1), (5120, 34816, 80, 80, 2, 0)]
        for Kd, N, T, tt, mh, pair in shapes:
            pk = random_packed_int4(Kd, N, 128, dev)
            x = torch.randn(T, Kd, device=dev).half()
            out = torch.zeros(T, pk.n_pad, dtype=torch.float32, device=dev)
            run = lambda i=0: K.gemm_int4_tc(pk, x, out, epi=L.TC_EPI_STORE_F32, t_tile=tt, m_halves=mh, cta_pair=bool(pair))
            if timed:
                _report(f"gemm_int4 K={Kd} N={N} T={T} t_tile={tt} outputs/CTA={128 * mh}{' CTA pairs' if pair else ''}",
                        time_launches(run, 1, 6), bytes_=pk.nbytes(), flops=2.0 * T * Kd * N)
            else:
                _profiled(run, 1)
    else:
        w = (torch.randn(34816, 5120, device=dev) * 0.02).half()
        for T, tt in ((512, 512), (80, 80)):
            x = torch.randn(T, 5120, device=dev).half()
            out = torch.zeros(T, 34816, dtype=torch.float32, device=dev)
            run = lambda i=0: K.gemm_f16_tc(w, x, out, t_tile=tt)
            if timed:
                _report(f"gemm_dense K=5120 N=34816 T={T}", time_launches(run, 1, 6), bytes_=w.numel() * 2,
                        flops=2.0 * T * 5120 * 34816)
            else:
                _profiled(run, 1)
    K.gemm_tc_check_status()


def case_attn_prefill(timed: bool):
    """Causal attention of a 512-row prompt (24 query / 4 KV heads of 256): the tcgen05 kernel and, with
    --time, the mma.sync many-row kernel on the same input."""
    dev = torch.device("cuda")
    nq, nkv, hd, T = 24, 4, 256, 512
    kc = torch.randn(1, T + 64, nkv, hd, device=dev).half()
    vc = torch.randn(1, T + 64, nkv, hd, device=dev).half()
    rm = K.make_rows([(0, i, i, i + 1, 0) for i in range(T)], dev)
    q = torch.randn(T, 2 * nq * hd, device=dev).half()
    out = torch.zeros(T, nq * hd, dtype=torch.float16, device=dev)
    run = lambda i=0: K.attn_prefill_tc(q, rm, kc, vc, nq, nkv, hd, gate_off=nq * hd, out=out)
    flops = 2.0 * 2.0 * nq * hd * T * (T + 1) / 2
    if timed:
        _report("attn_prefill tcgen05", time_launches(run, 1, 6), flops=flops)
        seq_rows = torch.tensor([0, T], dtype=torch.int32, device=dev)
        run2 = lambda i=0: K.attn_rows(q, rm, seq_rows, kc, vc, nq, nkv, hd, gate_off=nq * hd, splits=1, out=out)
        _report("attn_prefill mma.sync", time_launches(run2, 1, 6), flops=flops)
    else:
        _profiled(run, 1)


def case_attn(which: str, timed: bool):
    """attn_decode: 1 row, ctx 4096.  attn_rows: 80 rows (16 sequences x 5 draft rows), ctx 4096."""
    if which == "attn_prefill":
        return case_attn_prefill(timed)
    dev = torch.device("cuda")
    nq, nkv, hd, ctx = 24, 4, 256, 4096
    n_seq, per = (1, 1) if which == "attn_decode" else (16, 5)
    kc = torch.randn(n_seq, ctx + 64, nkv, hd, device=dev).half()
    vc = torch.randn(n_seq, ctx + 64, nkv, hd, device=dev).half()
    rows = [(s, ctx + i, ctx + i, ctx, (1 << (i + 1)) - 1) for s in range(n_seq) for i in range(per)]
    rm = K.make_rows(rows, dev)
    q = torch.randn(len(rows), 2 * nq * hd, device=dev).half()
    if which == "attn_rows":
        seq_rows = torch.arange(0, n_seq * per + 1, per, dtype=torch.int32, device=dev)
        run = lambda i=0: K.attn_rows(q, rm, seq_rows, kc, vc, nq, nkv, hd, gate_off=nq * hd, splits=2)
    else:
        run = lambda i=0: K.decode_attn(q, rm, kc, vc, nq, nkv, hd, gate_off=nq * hd, splits=16)
    if timed:
        _report(which, time_launches(run, 1, 6), bytes_=2.0 * n_seq * ctx * nkv * hd * 2)
    else:
        _profiled(run, 1)


def case_spec_step(timed: bool):
    """One 80-row verify-and-commit step of the 27B model (16 sequences x ctx 4096 x 4 drafts) on
    synthetic state; prints the step time.  Holds the whole model (about 22 GB): for launch lists
    (one pass per kernel) only, not for multi-pass captures."""
    from ..config import EngineConfig, qwen35_27b
    from ..engine.engine import InferenceEngine
    B, ctx, D = 16, 4096, 4
    eng = InferenceEngine(qwen35_27b(), max_seq_len=ctx + 64, max_batch=B,
                          engine_config=EngineConfig(max_step_rows=B * (D + 1)))
    eng.init_random(0)
    eng._ensure_driver()
    eng.states.kv.k.normal_(0, 0.5)
    eng.states.kv.v.normal_(0, 0.5)
    eng.states.dn.S.normal_(0, 0.05)
    drafts = [[1, 2, 3, 4] for _ in range(B)]
    parents = [list(range(-1, D - 1)) for _ in range(B)]

    def step():
        eng.states.seqs[:, 0] = ctx
        eng.states.seqs[:, 1] = 5
        eng.spec_step(drafts, parents, list(range(B)), sync=False)
    step(); step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.cudart().cudaProfilerStart()
    e0.record(); step(); e1.record()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    print(f"spec_step 80 rows: {e0.elapsed_time(e1):.2f} ms", flush=True)


def case_prefill(timed: bool):
    """pp512 of the 27B model at TP=1 (whole model resident: launch lists only)."""
    from ..config import qwen35_27b
    from ..engine.engine import InferenceEngine
    cfg = qwen35_27b()
    eng = InferenceEngine(cfg, max_seq_len=1024)
    eng.init_random(0)
    toks = torch.randint(0, cfg.vocab_size, (512,), generator=torch.Generator().manual_seed(1)).tolist()
    eng.prefill_tokens(toks[:64])
    eng.reset()
    eng.prefill_tokens(toks)
    eng.reset()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.cudart().cudaProfilerStart()
    e0.record(); eng.prefill_tokens(toks); e1.record()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    print(f"pp512: {e0.elapsed_time(e1):.2f} ms", flush=True)


def case_decode_step(timed: bool):
    """One eager decode step of the 27B model at TP=1 after a 128-token prompt (launch lists only)."""
    from ..config import qwen35_27b
    from ..engine.engine import InferenceEngine
    cfg = qwen35_27b()
    eng = InferenceEngine(cfg, max_seq_len=1024)
    eng.init_random(0)
    eng.prefill_tokens(torch.randint(0, cfg.vocab_size, (128,), generator=torch.Generator().manual_seed(1)).tolist())
    eng.decode_tokens(4, graph=False)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    eng.decode_tokens(1, graph=False)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()


def case_linear_q8(timed: bool):
    """W8A8 and W4A8 products of the gate_up shape (K 5120, N 34816) at 1, 8 and 64 rows."""
    dev = torch.device("cuda")
    Kd, N = 5120, 34816
    w8 = [torch.randint(-128, 128, (N, Kd), dtype=torch.int8, device=dev) for _ in range(2)]     # 2 x 178 MB > L2
    sw = torch.rand(N, device=dev) * 0.01
    w4 = [torch.randint(-2**31, 2**31 - 1, (N, Kd // 8), dtype=torch.int32, device=dev) for _ in range(3)]
    gs = (torch.rand(Kd // 128, N, device=dev) * 0.01).half()
    for T in (1, 8, 64):
        x = torch.randn(T, Kd, device=dev).half()
        xq, sx = K.act_quant_int8(x)
        r8 = lambda i=0: K.linear_w8a8(w8[i % 2], sw, xq, sx, out_dtype=torch.float16)
        r4 = lambda i=0: K.linear_w4a8(w4[i % 3], gs, xq, sx, out_dtype=torch.float16)
        if timed:
            _report(f"linear_w8a8 T={T}", time_launches(r8, 2, 8), bytes_=N * Kd, flops=2.0 * T * Kd * N)
            _report(f"linear_w4a8 T={T}", time_launches(r4, 3, 9), bytes_=N * Kd / 2, flops=2.0 * T * Kd * N)
            _report(f"act_quant T={T}", time_launches(lambda i=0: K.act_quant_int8(x), 1, 8))
        else:
            _profiled(r8, 1)
            _profiled(r4, 1)


def case_deltanet(which: str, timed: bool):
    from .microbench_deltanet import run_case
    run_case(which, timed, _profiled, _report)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--time", action="store_true")
    a = ap.parse_args()
    if a.case.startswith("gemv"):
        case_gemv(a.case, a.time)
    elif a.case.startswith("gemm"):
        case_gemm(a.case, a.time)
    elif a.case.startswith("attn"):
        case_attn(a.case, a.time)
    elif a.case == "spec_step":
        case_spec_step(a.time)
    elif a.case == "prefill":
        case_prefill(a.time)
    elif a.case == "decode_step":
        case_decode_step(a.time)
    elif a.case == "linear_q8":
        case_linear_q8(a.time)
    elif a.case.startswith("deltanet"):
        case_deltanet(a.case, a.time)
    else:
        raise SystemExit(f"unknown case {a.case}")
    print("ok")


if __name__ == "__main__":
    main()
