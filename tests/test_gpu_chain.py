"""The persistent projection-chain kernel (csrc/chain.cu) against a plain PyTorch fp32 reference of
the same four projections, and against the stand-alone GEMV path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-12))


def _rms(h, w, eps=1e-6):
    return (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * w.float()).half().float()


def _layer(K0, H, F, N3, g, rows, seed, zeros=True):
    from mi50grad_b200.ops.packing import interleave_gate_up, pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    gen = torch.Generator().manual_seed(seed)
    d = _dev()
    mk = lambda K, N: random_int4_linear(K, N, g, gen)
    o, gate, up, down, nxt = mk(K0, H), mk(H, F), mk(H, F), mk(F, H), mk(H, N3)
    if zeros:
        for l in (o, gate, up, down, nxt):
            l.zeros = torch.randint(0, 16, l.zeros.shape, generator=gen).half()
    x0 = torch.randn(rows, K0, generator=gen).half()
    h0 = torch.randn(rows, H, generator=gen)
    w1 = (torch.rand(H, generator=gen) + 0.5).half()
    w3 = (torch.rand(H, generator=gen) + 0.5).half()
    # fp32 reference with the kernel's fp16 rounding points (normalised input, SiLU output)
    h1 = h0 + x0.float() @ o.dense().t()
    xn1 = _rms(h1, w1)
    act = (torch.nn.functional.silu(xn1 @ gate.dense().t()) * (xn1 @ up.dense().t())).half().float()
    h2 = h1 + act @ down.dense().t()
    out = _rms(h2, w3) @ nxt.dense().t()
    pk = dict(o=pack_int4(o, d), gu=pack_int4(interleave_gate_up(gate.to(d), up.to(d)), d), down=pack_int4(down, d),
              nxt=pack_int4(nxt, d))
    return pk, x0.to(d), h0.to(d), w1.to(d), w3.to(d), dict(h1=h1, act=act, h2=h2, out=out)


@pytest.mark.parametrize("K0,H,F,N3,g,rows", [
    (256, 256, 704, 384, 128, 1),        # tiny model widths; F is padded to 768
    (512, 1024, 2176, 1280, 128, 3),
    (768, 640, 1408, 512, 32, 2),        # group 32
    (6144, 5120, 17408, 16384, 128, 1),  # the 27B decode shapes
    (768, 5120, 2176, 2048, 128, 8),     # the 27B shapes of one of 8 ranks, 8 rows
])
def test_chain_four_projections(K0, H, F, N3, g, rows):
    from mi50grad_b200.ops import kernels as K
    from mi50grad_b200.ops import lib as L
    pk, x0, h0, w1, w3, ref = _layer(K0, H, F, N3, g, rows, K0 + F)
    d = _dev()
    Fp = pk["gu"].n_pad // 2
    assert pk["down"].K == F
    np64 = -(-H // 64)
    h = h0.clone()
    ss = torch.zeros(rows, np64, device=d)
    act = torch.zeros(rows, Fp, dtype=torch.float16, device=d)
    out = torch.zeros(rows, N3, dtype=torch.float16, device=d)
    ops = [
        K.chain_op(pk["o"], x=x0, mode=L.EPI_FINISH, fin_flags=L.FIN_NO_COMM, h=h, ss_part=ss),
        K.chain_op(pk["gu"], ln=K.lazy_norm(h, ss, w1), mode=L.EPI_SILU_PAIR, out=act, n_valid=Fp),
        K.chain_op(pk["down"], x=act, mode=L.EPI_FINISH, fin_flags=L.FIN_NO_COMM, h=h, ss_part=ss),
        K.chain_op(pk["nxt"], ln=K.lazy_norm(h, ss, w3), out=out),
    ]
    # `down` reads F columns of a buffer with row stride Fp
    ops[2].ldx = Fp
    bufs = K.chain_scratch(ops, rows, d)
    K.chain(ops, rows, bufs)
    torch.cuda.synchronize()
    assert _rel(act[:, :F].cpu(), ref["act"]) < 4e-3
    assert _rel(h.cpu(), ref["h2"]) < 2e-3
    assert torch.allclose(ss.sum(-1).cpu(), ref["h2"].pow(2).sum(-1), rtol=2e-3)
    assert _rel(out.cpu(), ref["out"]) < 5e-3
    assert bufs.counters[:2].tolist() == [0, 1]                # departures cleared, one launch counted
    # a second launch on the same buffers (counters reused) gives the same bits
    h_b, out_a = h0.clone(), out.clone()
    ops[0] = K.chain_op(pk["o"], x=x0, mode=L.EPI_FINISH, fin_flags=L.FIN_NO_COMM, h=h_b, ss_part=ss)
    ops[1] = K.chain_op(pk["gu"], ln=K.lazy_norm(h_b, ss, w1), mode=L.EPI_SILU_PAIR, out=act, n_valid=Fp)
    ops[2] = K.chain_op(pk["down"], x=act, mode=L.EPI_FINISH, fin_flags=L.FIN_NO_COMM, h=h_b, ss_part=ss)
    ops[2].ldx = Fp
    ops[3] = K.chain_op(pk["nxt"], ln=K.lazy_norm(h_b, ss, w3), out=out)
    K.chain(ops, rows, bufs)
    torch.cuda.synchronize()
    assert torch.equal(out, out_a) and torch.equal(h_b, h)


def test_chain_matches_standalone_gemv_and_deferred_flags():
    """One projection per launch form, and the deferred_consistent epilogue flags."""
    from mi50grad_b200.ops import kernels as K
    from mi50grad_b200.ops import lib as L
    rows, K0, H = 2, 512, 1024
    pk, x0, h0, w1, w3, ref = _layer(K0, H, 704, 256, 128, rows, 3)
    d = _dev()
    np64 = H // 64
    # single store projection == the stand-alone kernel up to summation order
    out_c = torch.zeros(rows, H, dtype=torch.float32, device=d)
    out_g = torch.zeros(rows, H, dtype=torch.float32, device=d)
    op = K.chain_op(pk["o"], x=x0, mode=L.EPI_STORE_F32, out=out_c)
    bufs = K.chain_scratch([op], rows, d)
    K.chain([op], rows, bufs)
    K.gemv(pk["o"], x0, out=out_g, mode=L.EPI_STORE_F32)
    assert _rel(out_c.cpu(), out_g.cpu()) < 1e-4
    # attention partial kept aside (h untouched), then added to the FFN partial
    h = h0.clone()
    h_tmp, extra = torch.zeros_like(h), torch.zeros_like(h)
    ss = torch.zeros(rows, np64, device=d)
    y = (ref["h1"] - h0.cpu())
    op1 = K.chain_op(pk["o"], x=x0, mode=L.EPI_FINISH, fin_flags=L.FIN_NO_COMM | L.FIN_NO_H_WRITE | L.FIN_SAVE_EXTRA,
                     h=h, hout=h_tmp, extra=extra, ss_part=ss)
    K.chain([op1], rows, bufs)
    assert torch.equal(h, h0) and _rel(extra.cpu(), y) < 1e-4 and _rel(h_tmp.cpu(), ref["h1"]) < 1e-4
    op2 = K.chain_op(pk["o"], x=x0, mode=L.EPI_FINISH, fin_flags=L.FIN_NO_COMM | L.FIN_ADD_EXTRA, h=h, extra=extra,
                     ss_part=ss)
    K.chain([op2], rows, bufs)
    assert _rel(h.cpu(), h0.cpu() + 2 * y) < 1e-4


def test_chain_refuses_projections_that_do_not_feed_one_another():
    """Two projections of one launch must be producer and consumer: anything else is refused by the
    wrapper before a launch (the step driver then issues them as separate GEMV launches)."""
    from mi50grad_b200.ops import kernels as K
    from mi50grad_b200.ops.packing import random_packed_int4
    d = _dev()
    pk = random_packed_int4(512, 128, 128, d)
    x = torch.zeros(2, 512, dtype=torch.float16, device=d)
    out1 = torch.zeros(2, 128, dtype=torch.float16, device=d)
    out2 = torch.zeros(2, 128, dtype=torch.float16, device=d)
    ops = [K.chain_op(pk, x=x, out=out1), K.chain_op(pk, x=x, out=out2)]
    bufs = K.chain_scratch(ops, 2, d)
    with pytest.raises(ValueError):
        K.chain(ops, 2, bufs)
    K.chain(ops[:1], 2, bufs)                  # each alone is fine
    torch.cuda.synchronize()
