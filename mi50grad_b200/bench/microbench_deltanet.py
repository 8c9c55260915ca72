"""DeltaNet kernel cases for `bench.profile_cases` (27B head counts: 16 key / 48 value heads of 128)."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .microbench import time_launches


def run_case(which: str, timed: bool, profiled, report):
    dev = torch.device("cuda")
    dk = dv = 128
    nk, nv, H = 16, 48, 5120
    kd, vd = nk * dk, nv * dv
    conv_dim = 2 * kd + vd
    T = 512 if which == "deltanet_chunk" else 1
    g = torch.Generator(device=dev).manual_seed(0)
    proj = torch.randn(T, conv_dim + vd, device=dev, generator=g).half()
    conv_w = (torch.randn(conv_dim, 4, device=dev, generator=g) * 0.3).half()
    A_log = torch.rand(nv, device=dev, generator=g) * 1.5 - 1.0
    dt_bias = (torch.randn(nv, device=dev, generator=g) * 0.5).half()
    norm_w = (torch.rand(dv, device=dev, generator=g) + 0.5).half()
    state = torch.randn(1, nv, dk, dv, device=dev, generator=g) * 0.1
    conv_state = torch.zeros(1, nv, dv // 32, 2 * dk + 32, 3, dtype=torch.float16, device=dev)
    xn = torch.randn(T, H, device=dev, generator=g).half()
    wa = (torch.randn(nv, H, device=dev, generator=g) * 0.02).half()
    wb = (torch.randn(nv, H, device=dev, generator=g) * 0.02).half()
    rows = K.make_rows([(0, 0, 0, 0, 1)] * T, dev)
    seq_rows = torch.tensor([0, T], dtype=torch.int32, device=dev)
    offs = (0, kd, 2 * kd, conv_dim, -1, -1)
    if which == "deltanet_chunk":
        ab = K.ab_proj(xn, wa, wb)
        if timed:
            # the scan alone, with the q / k pre-pass, and with both pre-passes (their launches included)
            for mode in (0, 1, 2):
                run = lambda i=0: K.deltanet_chunk(proj, offs, ab, conv_w, conv_state, state, A_log, dt_bias, norm_w, rows,
                                                   seq_rows, nk, nv, dk, dv, prepass=mode)
                report(which + f" T={T} prepass={mode}", time_launches(run, 1, 6))
            return
        run = lambda i=0: K.deltanet_chunk(proj, offs, ab, conv_w, conv_state, state, A_log, dt_bias, norm_w, rows,
                                           seq_rows, nk, nv, dk, dv, prepass=2)
    else:
        run = lambda i=0: K.deltanet_step(proj, offs, conv_w, conv_state, state, A_log, dt_bias, norm_w, rows, seq_rows,
                                          nk, nv, dk, dv, xn=xn, wa=wa, wb=wb)
    if timed:
        flops = 0.0
        report(which + f" T={T}", time_launches(run, 1, 6), bytes_=2.0 * state.numel() * 4)
    else:
        profiled(run, 1)
