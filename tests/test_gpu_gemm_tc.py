"""tcgen05 INT4 GEMM against a PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-12))


@pytest.mark.parametrize("K,N,T,g", [(256, 128, 16, 128), (704, 200, 48, 128), (1024, 384, 512, 128),
                                    (2176, 640, 80, 128), (512, 256, 300, 32), (5120, 1024, 700, 128)])
def test_gemm_int4_tc_store(K, N, T, g):
    from mi50grad_b200.ops import kernels as Kn
    from mi50grad_b200.ops import lib as L
    from mi50grad_b200.ops.packing import pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(K + N + T)
    lin = random_int4_linear(K, N, g, gen)
    lin.zeros = torch.randint(0, 16, lin.zeros.shape, generator=gen).half()
    x = torch.randn(T, K, generator=gen).half()
    ref = x.float() @ lin.dense().t()
    pk = pack_int4(lin, dev)
    out = torch.full((T, N), float("nan"), dtype=torch.float16, device=dev)
    Kn.gemm_int4_tc(pk, x.to(dev), out)
    torch.cuda.synchronize()
    Kn.gemm_tc_check_status()
    assert _rel(out.cpu(), ref) < 3e-3
    out32 = torch.zeros(T, N, dtype=torch.float32, device=dev)
    Kn.gemm_int4_tc(pk, x.to(dev), out32, epi=L.TC_EPI_STORE_F32)
    Kn.gemm_int4_tc(pk, x.to(dev), out32, epi=L.TC_EPI_RESID_F32)
    torch.cuda.synchronize()
    Kn.gemm_tc_check_status()
    assert _rel(out32.cpu(), 2 * ref) < 2e-3


@pytest.mark.parametrize("K,N,T,ks,g", [(1024, 384, 512, 3, 128), (2176, 640, 80, 4, 128), (704, 200, 48, 2, 128),
                                         (512, 256, 300, 8, 32), (5120, 256, 512, 5, 128)])
def test_gemm_int4_tc_split_k_adds_into_the_residual(K, N, T, ks, g):
    """Several CTAs per output tile, each over a slice of K, add their partial products atomically."""
    from mi50grad_b200.ops import kernels as Kn
    from mi50grad_b200.ops import lib as L
    from mi50grad_b200.ops.packing import pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(K + N + T + ks)
    lin = random_int4_linear(K, N, g, gen)
    lin.zeros = torch.randint(0, 16, lin.zeros.shape, generator=gen).half()
    x = torch.randn(T, K, generator=gen).half()
    h0 = torch.randn(T, N, generator=gen)
    ref = h0 + x.float() @ lin.dense().t()
    pk = pack_int4(lin, dev)
    out = h0.to(dev).clone()
    Kn.gemm_int4_tc(pk, x.to(dev), out, epi=L.TC_EPI_RESID_F32, k_splits=ks)
    torch.cuda.synchronize()
    Kn.gemm_tc_check_status()
    assert _rel(out.cpu(), ref) < 2e-3


@pytest.mark.parametrize("K,N,T,g,ks", [(1024, 512, 512, 128, 1), (2176, 768, 80, 128, 1), (5120, 1024, 700, 128, 1),
                                         (512, 256, 300, 32, 1), (704, 256, 48, 128, 1), (2048, 512, 512, 128, 3)])
def test_gemm_int4_tc_256_output_tiles(K, N, T, g, ks):
    """CTAs that own 256 outputs as two accumulators sharing each activation tile: store, fp32 store, residual
    add (also with split-K)."""
    from mi50grad_b200.ops import kernels as Kn
    from mi50grad_b200.ops import lib as L
    from mi50grad_b200.ops.packing import pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(K + N + T + 1)
    lin = random_int4_linear(K, N, g, gen)
    lin.zeros = torch.randint(0, 16, lin.zeros.shape, generator=gen).half()
    x = torch.randn(T, K, generator=gen).half()
    ref = x.float() @ lin.dense().t()
    pk = pack_int4(lin, dev)
    assert pk.n_pad % 256 == 0
    out = torch.full((T, N), float("nan"), dtype=torch.float16, device=dev)
    Kn.gemm_int4_tc(pk, x.to(dev), out, m_halves=2)
    torch.cuda.synchronize()
    Kn.gemm_tc_check_status()
    assert _rel(out.cpu(), ref) < 3e-3
    h0 = torch.randn(T, N, generator=gen)
    out32 = h0.to(dev).clone()
    Kn.gemm_int4_tc(pk, x.to(dev), out32, epi=L.TC_EPI_RESID_F32, k_splits=ks, m_halves=2)
    torch.cuda.synchronize()
    Kn.gemm_tc_check_status()
    assert _rel(out32.cpu(), h0 + ref) < 2e-3


@pytest.mark.parametrize("K,N,T,tt", [(1024, 512, 512, 256), (2176, 768, 256, 256), (5120, 1024, 768, 256),
                                      (1024, 512, 512, 512), (5120, 1280, 1024, 512)])
def test_gemm_int4_tc_cta_pairs(K, N, T, tt):
    """Adjacent output tiles as CTA pairs: cta_group::2 MMAs, each CTA loading its half of the token operand."""
    from mi50grad_b200.ops import kernels as Kn
    from mi50grad_b200.ops import lib as L
    from mi50grad_b200.ops.packing import pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(K + N + T + 2)
    lin = random_int4_linear(K, N, 128, gen)
    lin.zeros = torch.randint(0, 16, lin.zeros.shape, generator=gen).half()
    x = torch.randn(T, K, generator=gen).half()
    ref = x.float() @ lin.dense().t()
    pk = pack_int4(lin, dev)
    out32 = torch.zeros(T, N, dtype=torch.float32, device=dev)
    Kn.gemm_int4_tc(pk, x.to(dev), out32, epi=L.TC_EPI_STORE_F32, t_tile=tt, cta_pair=True)
    torch.cuda.synchronize()
    Kn.gemm_tc_check_status()
    assert _rel(out32.cpu(), ref) < 2e-3


def test_gemm_int4_tc_silu_pair_256_output_tiles():
    from mi50grad_b200.ops import kernels as Kn
    from mi50grad_b200.ops import lib as L
    from mi50grad_b200.ops.packing import interleave_gate_up, pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(6)
    K, F, T = 512, 640, 300
    gate, up = random_int4_linear(K, F, 128, gen), random_int4_linear(K, F, 128, gen)
    x = torch.randn(T, K, generator=gen).half()
    ref = torch.nn.functional.silu(x.float() @ gate.dense().t()) * (x.float() @ up.dense().t())
    pk = pack_int4(interleave_gate_up(gate, up), dev)
    assert pk.n_pad % 256 == 0
    out = torch.zeros(T, pk.n_pad // 2, dtype=torch.float16, device=dev)
    Kn.gemm_int4_tc(pk, x.to(dev), out, epi=L.TC_EPI_SILU_PAIR, m_halves=2)
    torch.cuda.synchronize()
    Kn.gemm_tc_check_status()
    assert _rel(out[:, :F].cpu(), ref) < 4e-3


def test_gemm_int4_tc_silu_pair():
    from mi50grad_b200.ops import kernels as Kn
    from mi50grad_b200.ops import lib as L
    from mi50grad_b200.ops.packing import interleave_gate_up, pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(5)
    K, F, T = 512, 704, 100
    gate, up = random_int4_linear(K, F, 128, gen), random_int4_linear(K, F, 128, gen)
    x = torch.randn(T, K, generator=gen).half()
    ref = torch.nn.functional.silu(x.float() @ gate.dense().t()) * (x.float() @ up.dense().t())
    pk = pack_int4(interleave_gate_up(gate, up), dev)
    out = torch.zeros(T, pk.n_pad // 2, dtype=torch.float16, device=dev)
    Kn.gemm_int4_tc(pk, x.to(dev), out, epi=L.TC_EPI_SILU_PAIR)
    torch.cuda.synchronize()
    Kn.gemm_tc_check_status()
    assert _rel(out[:, :F].cpu(), ref) < 4e-3


@pytest.mark.parametrize("T,N,K", [(80, 1000, 256), (16, 128, 5120), (300, 777, 1024)])
def test_gemm_f16_tc_dense_weights(T, N, K):
    g = torch.Generator(device="cuda").manual_seed(T + N)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).half()
    x = torch.randn(T, K, device="cuda", generator=g).half()
    out = torch.zeros(T, -(-N // 4) * 4, dtype=torch.float32, device="cuda")
    from mi50grad_b200.ops import kernels as K_
    K_.gemm_f16_tc(w, x, out)
    K_.gemm_tc_check_status()
    ref = x.float() @ w.float().t()
    err = (out[:, :N] - ref).abs().max().item()
    assert err < 2e-3 * max(1.0, ref.abs().max().item()), err
