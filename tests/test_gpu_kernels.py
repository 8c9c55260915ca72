"""Each CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-12))


@pytest.fixture(scope="module")
def K():
    from mi50grad_b200.ops import kernels
    return kernels


@pytest.mark.parametrize("Kdim,N,rows,g,ks", [
    (256, 128, 1, 128, None), (704, 200, 3, 128, None), (5120, 1024, 1, 128, None),
    (5120, 1024, 8, 128, 3), (2176, 5120, 2, 128, None), (768, 640, 5, 32, 2), (6144, 5120, 1, 128, 6),
])
def test_gemv_int4_store(K, Kdim, N, rows, g, ks):
    from mi50grad_b200.ops.packing import pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    gen = torch.Generator().manual_seed(Kdim + N)
    lin = random_int4_linear(Kdim, N, g, gen)
    lin.zeros = torch.randint(0, 16, lin.zeros.shape, generator=gen).half()
    x = torch.randn(rows, Kdim, generator=gen).half()
    ref = x.float() @ lin.dense().t()
    pk = pack_int4(lin, _dev())
    out = torch.zeros(rows, N, dtype=torch.float16, device=_dev())
    K.gemv(pk, x.to(_dev()), out=out, k_splits=ks)
    torch.cuda.synchronize()
    assert _rel(out.cpu(), ref) < 2e-3
    out32 = torch.zeros(rows, N, dtype=torch.float32, device=_dev())
    from mi50grad_b200.ops import lib as L
    K.gemv(pk, x.to(_dev()), out=out32, mode=L.EPI_STORE_F32, k_splits=ks)
    assert _rel(out32.cpu(), ref) < 2e-4


def test_gemv_int4_row_shard_with_group_offset(K):
    from mi50grad_b200.ops.packing import pack_int4
    from mi50grad_b200.parallel.sharding import slice_in
    from mi50grad_b200.utils.quant import random_int4_linear
    gen = torch.Generator().manual_seed(5)
    lin = slice_in(random_int4_linear(704, 256, 128, gen), 352, 704)
    assert lin.group_offset == 96
    x = torch.randn(2, 352, generator=gen).half()
    ref = x.float() @ lin.dense().t()
    out = torch.zeros(2, 256, dtype=torch.float16, device=_dev())
    K.gemv(pack_int4(lin, _dev()), x.to(_dev()), out=out)
    assert _rel(out.cpu(), ref) < 2e-3


def test_gemv_int4_awq_no_zero(K):
    from mi50grad_b200.ops.packing import pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    gen = torch.Generator().manual_seed(6)
    lin = random_int4_linear(512, 384, 128, gen, zeros=None)
    x = torch.randn(1, 512, generator=gen).half()
    out = torch.zeros(1, 384, dtype=torch.float16, device=_dev())
    K.gemv(pack_int4(lin, _dev()), x.to(_dev()), out=out)
    assert _rel(out.cpu(), x.float() @ lin.dense().t()) < 2e-3


@pytest.mark.parametrize("rows,F", [(1, 704), (4, 2176)])
def test_gemv_silu_pair(K, rows, F):
    from mi50grad_b200.ops import lib as L
    from mi50grad_b200.ops.packing import interleave_gate_up, pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    gen = torch.Generator().manual_seed(7)
    Kd = 256
    gate, up = random_int4_linear(Kd, F, 128, gen), random_int4_linear(Kd, F, 128, gen)
    x = torch.randn(rows, Kd, generator=gen).half()
    ref = torch.nn.functional.silu(x.float() @ gate.dense().t()) * (x.float() @ up.dense().t())
    pk = pack_int4(interleave_gate_up(gate, up), _dev())
    Fp = pk.n_pad // 2
    out = torch.full((rows, Fp), 7.0, dtype=torch.float16, device=_dev())
    K.gemv(pk, x.to(_dev()), out=out, mode=L.EPI_SILU_PAIR)
    assert _rel(out[:, :F].cpu(), ref) < 3e-3
    assert float(out[:, F:].abs().max()) == 0.0 if Fp > F else True


@pytest.mark.parametrize("rows,ks", [(1, None), (3, 4)])
def test_gemv_finish_local_residual_and_lazy_norm(K, rows, ks):
    """Row-parallel epilogue without exchange: h += y per tile, per-tile sums of squares;
    the consumer GEMV applies the RMSNorm while staging its input."""
    from mi50grad_b200.ops import lib as L
    from mi50grad_b200.ops.packing import pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    gen = torch.Generator().manual_seed(8)
    Kd, H = 1024, 5120
    lin = random_int4_linear(Kd, H, 128, gen)
    x = torch.randn(rows, Kd, generator=gen).half()
    h0 = torch.randn(rows, H, generator=gen)
    w = (torch.rand(H, generator=gen) + 0.5).half()
    y = x.float() @ lin.dense().t()
    h_ref = h0 + y
    xn_ref = h_ref * torch.rsqrt(h_ref.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    d = _dev()
    pk = pack_int4(lin, d)
    h = h0.to(d).clone()
    ss = K.gemv(pk, x.to(d), mode=L.EPI_FINISH, fin_flags=L.FIN_NO_COMM, h=h, k_splits=ks)
    assert _rel(h.cpu(), h_ref) < 1e-4
    assert ss.shape == (rows, 40)
    assert torch.allclose(ss.sum(-1).cpu(), h_ref.pow(2).sum(-1), rtol=1e-4)
    # consumer: INT4 and fp16 GEMVs reading the lazily normalised stream
    lin2 = random_int4_linear(H, 256, 128, gen)
    out = torch.zeros(rows, 256, dtype=torch.float16, device=d)
    K.gemv(pack_int4(lin2, d), None, out=out, ln=K.lazy_norm(h, ss, w.to(d)), rows=rows)
    assert _rel(out.cpu(), xn_ref.half().float() @ lin2.dense().t()) < 3e-3
    from mi50grad_b200.engine.engine import DeviceLinear
    wd = (torch.randn(300, H, generator=gen) * 0.05).half()
    out32 = torch.zeros(rows, 300, dtype=torch.float32, device=d)
    K.gemv(DeviceLinear(dense=wd.to(d)), None, out=out32, mode=L.EPI_STORE_F32, ln=K.lazy_norm(h, ss, w.to(d)),
           rows=rows)
    assert _rel(out32.cpu(), xn_ref.half().float() @ wd.float().t()) < 2e-3
    # deferred_consistent attention form: h untouched, h+y goes to a scratch stream, partial saved;
    # the following projection adds the saved partial to its own
    h2 = h0.to(d).clone()
    h_tmp = torch.zeros_like(h2)
    extra = torch.zeros(rows, H, dtype=torch.float32, device=d)
    K.gemv(pk, x.to(d), mode=L.EPI_FINISH, fin_flags=L.FIN_NO_COMM | L.FIN_NO_H_WRITE | L.FIN_SAVE_EXTRA,
           h=h2, hout=h_tmp, extra=extra)
    assert torch.equal(h2.cpu(), h0) and _rel(extra.cpu(), y) < 1e-4 and _rel(h_tmp.cpu(), h_ref) < 1e-4
    K.gemv(pk, x.to(d), mode=L.EPI_FINISH, fin_flags=L.FIN_NO_COMM | L.FIN_ADD_EXTRA, h=h2, extra=extra)
    assert _rel(h2.cpu(), h0 + 2 * y) < 1e-4


@pytest.mark.parametrize("N,Kd,rows", [(1000, 512, 1), (4096, 5120, 3), (300, 6144, 8)])
def test_gemv_f16(K, N, Kd, rows):
    from mi50grad_b200.engine.engine import DeviceLinear
    from mi50grad_b200.ops import lib as L
    gen = torch.Generator().manual_seed(9)
    w = (torch.randn(N, Kd, generator=gen) * 0.05).half()
    x = torch.randn(rows, Kd, generator=gen).half()
    ref = x.float() @ w.float().t()
    lin = DeviceLinear(dense=w.to(_dev()))
    out = torch.zeros(rows, N, dtype=torch.float32, device=_dev())
    K.gemv(lin, x.to(_dev()), out=out, mode=L.EPI_STORE_F32)
    assert _rel(out.cpu(), ref) < 1e-4
    out16 = torch.zeros(rows, N, dtype=torch.float16, device=_dev())
    K.gemv(lin, x.to(_dev()), out=out16, mode=L.EPI_STORE_F16)
    assert _rel(out16.cpu(), ref) < 2e-3


def test_add_rmsnorm_and_embed(K):
    gen = torch.Generator().manual_seed(10)
    d = _dev()
    H = 5120
    h0, delta = torch.randn(3, H, generator=gen), torch.randn(3, H, generator=gen)
    w = (torch.rand(H, generator=gen) + 0.5).half()
    h = h0.to(d).clone()
    xn = K.add_rmsnorm(h, w.to(d), delta.to(d))
    hr = h0 + delta
    ref = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert _rel(h.cpu(), hr) < 1e-6 and _rel(xn.cpu(), ref) < 2e-3
    embed = (torch.randn(50, H, generator=gen) * 0.1).half()
    rows = K.make_rows([(0, 0, 0, 0, 1), (1, 0, 0, 0, 1)], d)
    seqs = torch.tensor([[0, 7, 0, 0], [0, 9, 0, 0]], dtype=torch.int32, device=d)
    row_tokens = torch.tensor([-1, 33], dtype=torch.int32, device=d)
    hh = torch.zeros(2, H, device=d)
    xx = torch.zeros(2, H, dtype=torch.float16, device=d)
    ssp = torch.full((2, 40), 7.0, device=d)
    K.embed_rmsnorm(embed.to(d), row_tokens, rows, seqs, w.to(d), hh, xx, ssp)
    e = embed[[7, 33]].float()
    assert torch.equal(hh.cpu(), e)
    assert torch.allclose(ssp[:, 0].cpu(), e.pow(2).sum(-1), rtol=1e-5) and float(ssp[:, 1:].abs().max()) == 0
    assert _rel(xx.cpu(), e * torch.rsqrt(e.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()) < 2e-3


@pytest.mark.parametrize("hd,rot,style", [(256, 64, "interleaved"), (64, 16, "interleaved"), (128, 32, "half")])
def test_qknorm_rope_cachew(K, hd, rot, style):
    from mi50grad_b200.config import QwenConfig
    from mi50grad_b200.models import oracle as O
    gen = torch.Generator().manual_seed(11)
    d = _dev()
    nq, nkv, rows, max_seq = 6, 2, 3, 32
    cfg = QwenConfig(head_dim=hd, partial_rotary_factor=rot / hd, rope_style=style)
    qkv = torch.randn(rows, 2 * nq * hd + 2 * nkv * hd, generator=gen).half()
    qn, kn = (torch.rand(hd, generator=gen) + 0.5).half(), (torch.rand(hd, generator=gen) + 0.5).half()
    pos = torch.tensor([5, 0, 17])
    cos, sin = O.rope_tables(cfg, torch.arange(max_seq))
    meta = K.make_rows([(1, 5, 5, 5, 1), (0, 0, 3, 0, 1), (1, 17, 9, 9, 1)], d)
    kc = torch.zeros(2, max_seq, nkv, hd, dtype=torch.float16, device=d)
    vc = torch.zeros_like(kc)
    buf = qkv.to(d).clone()
    K.qknorm_rope_cachew(buf, meta, qn.to(d), kn.to(d), cos.to(d), sin.to(d), kc, vc, nq, nkv, hd, rot,
                         interleaved=(style == "interleaved"))
    q = qkv[:, :nq * hd].float().view(rows, nq, hd)
    k = qkv[:, 2 * nq * hd:2 * nq * hd + nkv * hd].float().view(rows, nkv, hd)
    v = qkv[:, 2 * nq * hd + nkv * hd:].float().view(rows, nkv, hd)
    qr = O.apply_rope(O.rmsnorm(q, qn, 1e-6), cos[pos], sin[pos], style)
    kr = O.apply_rope(O.rmsnorm(k, kn, 1e-6), cos[pos], sin[pos], style)
    assert _rel(buf[:, :nq * hd].cpu().view(rows, nq, hd), qr) < 2e-3
    assert torch.equal(buf[:, nq * hd:].cpu(), qkv[:, nq * hd:])          # gate, K, V untouched in place
    for r, (s, slot) in enumerate([(1, 5), (0, 3), (1, 9)]):
        assert _rel(kc[s, slot].cpu(), kr[r]) < 2e-3
        assert torch.equal(vc[s, slot].cpu(), v[r].half())


@pytest.mark.parametrize("hd,nq,nkv,splits", [(256, 6, 1, 4), (256, 24, 4, 1), (64, 4, 2, 3), (128, 3, 1, 8), (256, 24, 4, 32)])
def test_decode_attn(K, hd, nq, nkv, splits):
    from mi50grad_b200.models import oracle as O
    gen = torch.Generator().manual_seed(12)
    d = _dev()
    max_seq, nseq = 1200, 2
    kc = torch.randn(nseq, max_seq, nkv, hd, generator=gen).half()
    vc = torch.randn(nseq, max_seq, nkv, hd, generator=gen).half()
    # rows: plain decode at ctx 200 (seq 1), ctx 3 (seq 0), a draft node with a sparse ancestor mask, ctx 0
    entries = [(1, 1100, 1100, 1100, 1), (0, 3, 3, 3, 1), (1, 0, 0, 100, 0b1011), (0, 0, 0, 0, 1), (0, 300, 300, 300, 1)]
    rows = len(entries)
    q = torch.randn(rows, 2 * nq * hd, generator=gen).half()
    out = K.decode_attn(q.to(d), K.make_rows(entries, d), kc.to(d), vc.to(d), nq, nkv, hd, gate_off=nq * hd,
                        splits=splits)
    for r, (s, _, _, ctx, mask) in enumerate(entries):
        vis = list(range(ctx)) + [ctx + j for j in range(64) if (mask >> j) & 1]
        Kr, Vr = kc[s, vis].float(), vc[s, vis].float()
        o = O.attention(q[r:r + 1, :nq * hd].float().view(1, nq, hd), Kr, Vr,
                        torch.ones(1, len(vis), dtype=torch.bool))
        o = o * torch.sigmoid(q[r, nq * hd:].float().view(1, nq, hd))
        assert _rel(out[r].cpu().view(nq, hd), o[0]) < 3e-3, f"row {r}"


@pytest.mark.parametrize("hd,nq,nkv,splits", [(256, 6, 1, 1), (256, 24, 4, 3), (64, 4, 2, 1), (64, 6, 2, 4)])
def test_attn_rows_tensor_core(K, hd, nq, nkv, splits):
    """Many-row attention: a 40-row causal prompt chunk behind 5 cached tokens (three tiles, the last
    partial), a 6-node draft tree behind 137 cached tokens, and a single decode row."""
    from mi50grad_b200.models import oracle as O
    gen = torch.Generator().manual_seed(15)
    d = _dev()
    max_seq, nseq = 256, 3
    kc = torch.randn(nseq, max_seq, nkv, hd, generator=gen).half()
    vc = torch.randn(nseq, max_seq, nkv, hd, generator=gen).half()
    entries = [(0, 5 + i, 5 + i, 5 + i + 1, 0) for i in range(40)]
    anc = [0b1, 0b11, 0b101, 0b1011, 0b10011, 0b100101]
    entries += [(1, 137, 137 + i, 137, anc[i]) for i in range(6)]
    entries += [(2, 200, 200, 200, 1)]
    seq_rows = torch.tensor([0, 40, 46, 47], dtype=torch.int32)
    rows = len(entries)
    q = torch.randn(rows, 2 * nq * hd, generator=gen).half()
    out = K.attn_rows(q.to(d), K.make_rows(entries, d), seq_rows.to(d), kc.to(d), vc.to(d), nq, nkv, hd,
                      gate_off=nq * hd, splits=splits)
    for r, (s_, _, _, ctx, mask) in enumerate(entries):
        vis = list(range(ctx)) + [ctx + j for j in range(64) if (mask >> j) & 1]
        o = O.attention(q[r:r + 1, :nq * hd].float().view(1, nq, hd), kc[s_, vis].float(), vc[s_, vis].float(),
                        torch.ones(1, len(vis), dtype=torch.bool))
        o = o * torch.sigmoid(q[r, nq * hd:].float().view(1, nq, hd))
        assert _rel(out[r].cpu().view(nq, hd), o[0]) < 4e-3, f"row {r}"


@pytest.mark.parametrize("hd,nq,nkv,T,past", [(64, 4, 2, 40, 5), (64, 2, 1, 200, 0), (256, 6, 1, 130, 7),
                                              (256, 12, 2, 512, 0), (128, 4, 4, 300, 64)])
def test_attn_prefill_tcgen05(K, hd, nq, nkv, T, past):
    """Causal prompt attention on tcgen05: T rows of sequence 1 behind `past` cached tokens (partial row
    and slot tiles), against the fp32 reference, with the sigmoid output gate."""
    from mi50grad_b200.models import oracle as O
    gen = torch.Generator().manual_seed(31 + T)
    d = _dev()
    max_seq, nseq = 640, 2
    kc = torch.randn(nseq, max_seq, nkv, hd, generator=gen).half()
    vc = torch.randn(nseq, max_seq, nkv, hd, generator=gen).half()
    entries = [(1, past + i, past + i, past + i + 1, 0) for i in range(T)]
    q = torch.randn(T, 2 * nq * hd, generator=gen).half()
    out = K.attn_prefill_tc(q.to(d), K.make_rows(entries, d), kc.to(d), vc.to(d), nq, nkv, hd, gate_off=nq * hd)
    torch.cuda.synchronize()
    K.gemm_tc_check_status()
    worst = 0.0
    for r in list(range(0, T, 7)) + [T - 1]:
        ctx = past + r + 1
        o = O.attention(q[r:r + 1, :nq * hd].float().view(1, nq, hd), kc[1, :ctx].float(), vc[1, :ctx].float(),
                        torch.ones(1, ctx, dtype=torch.bool))
        o = o * torch.sigmoid(q[r, nq * hd:].float().view(1, nq, hd))
        worst = max(worst, _rel(out[r].cpu().view(nq, hd), o[0]))
    assert worst < 4e-3, worst


@pytest.mark.parametrize("dk,nk,nv,rows_per_seq,inkernel_ab", [(128, 2, 6, [1], True), (64, 2, 4, [3, 1], False),
                                                              (128, 1, 3, [5], False), (64, 1, 2, [2], "lazy")])
def test_deltanet_step(K, dk, nk, nv, rows_per_seq, inkernel_ab):
    from mi50grad_b200.models import oracle as O
    gen = torch.Generator().manual_seed(13)
    d = _dev()
    dv, H = dk, 512
    nseq = len(rows_per_seq)
    R = sum(rows_per_seq)
    kd, vd = nk * dk, nv * dv
    conv_dim = 2 * kd + vd
    ld = conv_dim + vd + 2 * nv
    proj = (torch.randn(R, ld, generator=gen)).half()
    conv_w = (torch.randn(conv_dim, 4, generator=gen) * 0.3).half()
    A_log = torch.rand(nv, generator=gen) * 1.5 - 1.0
    dt_bias = (torch.randn(nv, generator=gen) * 0.5).half()
    norm_w = (torch.rand(dv, generator=gen) + 0.5).half()
    S0 = torch.randn(nseq, nv, dk, dv, generator=gen) * 0.1
    hist0 = torch.randn(nseq, conv_dim, 3, generator=gen).half()
    hres = torch.randn(R, H, generator=gen) * 3
    wnorm = (torch.rand(H, generator=gen) + 0.5).half()
    xn = (hres * torch.rsqrt(hres.pow(2).mean(-1, keepdim=True) + 1e-6) * wnorm.float()).half() \
        if inkernel_ab == "lazy" else torch.randn(R, H, generator=gen).half()
    wa, wb = (torch.randn(nv, H, generator=gen) * 0.05).half(), (torch.randn(nv, H, generator=gen) * 0.05).half()
    if inkernel_ab:
        a_all = (xn.float() @ wa.float().t()).half().float()
        b_all = (xn.float() @ wb.float().t()).half().float()
        offs = (0, kd, 2 * kd, conv_dim, -1, -1)
    else:
        a_all, b_all = proj[:, conv_dim + vd:conv_dim + vd + nv].float(), proj[:, conv_dim + vd + nv:].float()
        offs = (0, kd, 2 * kd, conv_dim, conv_dim + vd, conv_dim + vd + nv)
    # private conv histories per (head, column block)
    CB, nch = dv // 32, 2 * dk + 32
    conv_state = torch.zeros(nseq, nv, CB, nch, 3, dtype=torch.float16)
    for j in range(nv):
        kh = j // (nv // nk)
        for cb in range(CB):
            ch = list(range(kh * dk, (kh + 1) * dk)) + list(range(kd + kh * dk, kd + (kh + 1) * dk)) + \
                list(range(2 * kd + j * dv + cb * 32, 2 * kd + j * dv + cb * 32 + 32))
            conv_state[:, j, cb] = hist0[:, ch]
    seq_rows = [0]
    entries = []
    for s, n in enumerate(rows_per_seq):
        entries += [(s, 0, 0, 0, 1)] * n
        seq_rows.append(seq_rows[-1] + n)
    state_d, conv_d = S0.to(d).clone(), conv_state.to(d).clone()
    out = K.deltanet_step(proj.to(d), offs, conv_w.to(d), conv_d, state_d, A_log.to(d), dt_bias.to(d),
                          norm_w.to(d), K.make_rows(entries, d), torch.tensor(seq_rows, dtype=torch.int32, device=d),
                          nk, nv, dk, dv, xn=xn.to(d) if inkernel_ab is True else None,
                          wa=wa.to(d) if inkernel_ab else None, wb=wb.to(d) if inkernel_ab else None,
                          ln=K.lazy_norm(hres.to(d), torch.cat([hres.pow(2).sum(-1, keepdim=True),
                                                                torch.zeros(R, 3)], 1).to(d), wnorm.to(d))
                          if inkernel_ab == "lazy" else None)
    for s in range(nseq):
        r0, r1 = seq_rows[s], seq_rows[s + 1]
        hist = hist0[s].clone()
        c = O.causal_conv1d(proj[r0:r1, :conv_dim].float(), hist, conv_w)
        n = r1 - r0
        qq = O.l2norm(c[:, :kd].reshape(n, nk, dk)) / math.sqrt(dk)
        kk = O.l2norm(c[:, kd:2 * kd].reshape(n, nk, dk))
        vv = c[:, 2 * kd:].reshape(n, nv, dv)
        rep = nv // nk
        g, beta = O.deltanet_gates(a_all[r0:r1], b_all[r0:r1], A_log, dt_bias)
        st = S0[s].clone()
        y = O.deltanet_recurrent(qq.repeat_interleave(rep, 1), kk.repeat_interleave(rep, 1), vv, g, beta, st)
        z = proj[r0:r1, conv_dim:conv_dim + vd].float().view(n, nv, dv)
        ref = O.gated_rmsnorm(y, z, norm_w).reshape(n, vd)
        assert _rel(out[r0:r1].cpu(), ref) < 4e-3, f"seq {s}"
        assert _rel(state_d[s].cpu(), st) < 1e-3
        # conv history of head 0 / block 0 ends with the last three inputs
        ch = list(range(0, dk))
        assert torch.equal(conv_d[s, 0, 0, :dk].cpu(), hist[ch].half())


@pytest.mark.parametrize("dk,nk,nv,rows_per_seq,prepass", [(128, 1, 3, [150], 0), (64, 2, 4, [70, 5, 64], 0),
                                                           (128, 2, 2, [512], 0), (128, 1, 3, [150], 1),
                                                           (64, 2, 4, [77], 1), (128, 2, 6, [512], 1),
                                                           (128, 1, 3, [150], 2), (64, 2, 4, [77], 2),
                                                           (128, 2, 6, [512], 2), (64, 1, 2, [32], 2)])
def test_deltanet_chunked_scan(K, dk, nk, nv, rows_per_seq, prepass):
    """Chunked scan == token-serial oracle (outputs, final state, conv history), with everything inside the
    scan (0), the q / k convolution and norms in a parallel pre-pass (1), and also the state-independent
    products and the triangle inverse of every chunk (2)."""
    from mi50grad_b200.models import oracle as O
    gen = torch.Generator().manual_seed(21)
    d = _dev()
    dv, H = dk, 256
    nseq, R = len(rows_per_seq), sum(rows_per_seq)
    kd, vd = nk * dk, nv * dv
    conv_dim = 2 * kd + vd
    proj = torch.randn(R, conv_dim + vd, generator=gen).half()
    conv_w = (torch.randn(conv_dim, 4, generator=gen) * 0.3).half()
    A_log = torch.rand(nv, generator=gen) * 1.5 - 1.0
    dt_bias = (torch.randn(nv, generator=gen) * 0.5).half()
    norm_w = (torch.rand(dv, generator=gen) + 0.5).half()
    S0 = torch.randn(nseq, nv, dk, dv, generator=gen) * 0.1
    hist0 = torch.randn(nseq, conv_dim, 3, generator=gen).half()
    xn = torch.randn(R, H, generator=gen).half()
    wa, wb = (torch.randn(nv, H, generator=gen) * 0.1).half(), (torch.randn(nv, H, generator=gen) * 0.1).half()
    ab = K.ab_proj(xn.to(d), wa.to(d), wb.to(d))
    ab_ref = torch.cat([xn.float() @ wa.float().t(), xn.float() @ wb.float().t()], 1)
    assert _rel(ab.cpu(), ab_ref) < 2e-3
    CB, nch = dv // 32, 2 * dk + 32
    conv_state = torch.zeros(nseq, nv, CB, nch, 3, dtype=torch.float16)
    for j in range(nv):
        kh = j // (nv // nk)
        for cb in range(CB):
            ch = list(range(kh * dk, (kh + 1) * dk)) + list(range(kd + kh * dk, kd + (kh + 1) * dk)) + \
                list(range(2 * kd + j * dv + cb * 32, 2 * kd + j * dv + cb * 32 + 32))
            conv_state[:, j, cb] = hist0[:, ch]
    seq_rows, entries = [0], []
    for s_, n in enumerate(rows_per_seq):
        entries += [(s_, 0, 0, 0, 1)] * n
        seq_rows.append(seq_rows[-1] + n)
    state_d, conv_d = S0.to(d).clone(), conv_state.to(d).clone()
    out = K.deltanet_chunk(proj.to(d), (0, kd, 2 * kd, conv_dim, -1, -1), ab, conv_w.to(d), conv_d, state_d,
                           A_log.to(d), dt_bias.to(d), norm_w.to(d), K.make_rows(entries, d),
                           torch.tensor(seq_rows, dtype=torch.int32, device=d), nk, nv, dk, dv, prepass=prepass)
    abh = ab.cpu().float()
    for s_ in range(nseq):
        r0, r1 = seq_rows[s_], seq_rows[s_ + 1]
        n = r1 - r0
        hist = hist0[s_].clone()
        c = O.causal_conv1d(proj[r0:r1, :conv_dim].float(), hist, conv_w)
        qq = O.l2norm(c[:, :kd].reshape(n, nk, dk)) / math.sqrt(dk)
        kk = O.l2norm(c[:, kd:2 * kd].reshape(n, nk, dk))
        vv = c[:, 2 * kd:].reshape(n, nv, dv)
        rep = nv // nk
        g, beta = O.deltanet_gates(abh[r0:r1, :nv], abh[r0:r1, nv:], A_log, dt_bias)
        st = S0[s_].clone()
        y = O.deltanet_recurrent(qq.repeat_interleave(rep, 1), kk.repeat_interleave(rep, 1), vv, g, beta, st)
        z = proj[r0:r1, conv_dim:].float().view(n, nv, dv)
        ref = O.gated_rmsnorm(y, z, norm_w).reshape(n, vd)
        assert _rel(out[r0:r1].cpu(), ref) < 4e-3, f"seq {s_}"
        assert _rel(state_d[s_].cpu(), st) < 2e-3
        assert torch.equal(conv_d[s_, 0, 0, :dk].cpu(), hist[:dk].half())


def test_deltanet_dry_run_keeps_state(K):
    gen = torch.Generator().manual_seed(14)
    d = _dev()
    dk = dv = 64
    nk, nv = 1, 2
    kd, vd = dk, nv * dv
    conv_dim = 2 * kd + vd
    proj = torch.randn(2, conv_dim + vd + 2 * nv, generator=gen).half().to(d)
    S = (torch.randn(1, nv, dk, dv, generator=gen) * 0.1).to(d)
    conv = torch.randn(1, nv, 2, 2 * dk + 32, 3, generator=gen).half().to(d)
    S0, conv0 = S.clone(), conv.clone()
    args = (proj, (0, kd, 2 * kd, conv_dim, conv_dim + vd, conv_dim + vd + nv),
            (torch.randn(conv_dim, 4, generator=gen) * 0.3).half().to(d), conv, S,
            torch.zeros(nv, device=d), torch.zeros(nv, dtype=torch.float16, device=d),
            torch.ones(dv, dtype=torch.float16, device=d), K.make_rows([(0, 0, 0, 0, 1)] * 2, d),
            torch.tensor([0, 2], dtype=torch.int32, device=d), nk, nv, dk, dv)
    a = K.deltanet_step(*args, commit=False).clone()
    assert torch.equal(S, S0) and torch.equal(conv, conv0)
    b = K.deltanet_step(*args, commit=True)
    assert torch.equal(a, b) and not torch.equal(S, S0)


def test_argmax_ties_and_blocks(K):
    gen = torch.Generator().manual_seed(15)
    d = _dev()
    logits = torch.randn(3, 248320, generator=gen)
    logits[1, 1000] = logits[1, 200000] = 50.0
    for blocks in (1, 16, 121):
        out = K.argmax(logits.to(d), vocab_offset=10, blocks=blocks)
        assert out.cpu().tolist() == [int(logits[0].argmax()) + 10, 1010, int(logits[2].argmax()) + 10]


def test_small_elementwise(K):
    gen = torch.Generator().manual_seed(16)
    d = _dev()
    g, u = torch.randn(1001, generator=gen).half(), torch.randn(1001, generator=gen).half()
    assert _rel(K.silu_mul(g.to(d), u.to(d)).cpu(), torch.nn.functional.silu(g.float()) * u.float()) < 2e-3
    x = g.to(d).clone()
    K.sigmoid_mul_(x, u.to(d))
    assert _rel(x.cpu(), g.float() * torch.sigmoid(u.float())) < 2e-3
    h = torch.randn(777, generator=gen)
    hd = h.to(d).clone()
    K.residual_add_(hd, g[:777].to(d))
    assert _rel(hd.cpu(), h + g[:777].float()) < 1e-6


@pytest.mark.parametrize("temp,top_k,top_p,pen", [(0.8, 50, 0.9, 1.3), (1.0, 5, 1.0, 1.0), (0.6, 0, 0.95, 1.1)])
def test_device_sampler_distribution_matches_host(K, temp, top_k, top_p, pen):
    """The kept candidates and their probabilities equal generate.sampler.filtered_probs; draws fall
    in the support and follow it."""
    import numpy as np
    from mi50grad_b200.generate.sampler import SamplingParams, filtered_probs
    d = _dev()
    gen = torch.Generator().manual_seed(33)
    V, rows = 5003, 3
    logits = torch.randn(rows, V, generator=gen) * 3.0
    logits[0, 17] = logits[0, 900] = 9.5                         # a tie among the top candidates
    past = torch.randint(0, V, (rows, 12), generator=gen).int()
    past[:, 3] = past[:, 4]                                       # duplicate entries count once
    n_past = torch.tensor([12, 5, 0], dtype=torch.int32)
    prm = SamplingParams(temperature=temp, top_k=top_k, top_p=top_p, repetition_penalty=pen)
    lg = logits.to(d).clone()
    tok, ids, probs = K.sample_top_p(lg, temp, top_k, top_p, pen, past.to(d), n_past.to(d), seed=7, debug=True)
    for r in range(rows):
        ref = filtered_probs(logits[r].numpy().copy(), prm, past[r, :int(n_past[r])].tolist())
        sup = np.nonzero(ref)[0]
        got_ids = ids[r].cpu().numpy()
        got_ids = got_ids[got_ids >= 0]
        assert sorted(got_ids.tolist()) == sorted(sup.tolist()), r
        gp = probs[r].cpu().numpy()[:len(got_ids)]
        assert np.allclose(gp, ref[got_ids], atol=2e-5), r
        assert int(tok[r]) in set(sup.tolist())
    # draws follow the distribution: 400 seeds on row 1
    ref = filtered_probs(logits[1].numpy().copy(), prm, past[1, :5].tolist())
    counts = {}
    for s in range(400):
        t = int(K.sample_top_p(logits[1:2].to(d).clone(), temp, top_k, top_p, pen, past[1:2].to(d), n_past[1:2].to(d),
                               seed=1000 + s)[0])
        counts[t] = counts.get(t, 0) + 1
    top = int(np.argmax(ref))
    assert abs(counts.get(top, 0) / 400.0 - ref[top]) < 0.1
