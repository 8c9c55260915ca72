"""INT8-activation linear layers against plain fp32 PyTorch (reference tests:
tests/test_w8a8_kernels.py, tests/test_w4a8_kernels.py)."""
import pytest
import torch

from mi50grad_b200.utils import quant as Q

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from mi50grad_b200.ops import kernels
    return kernels


def test_act_quant_rows(K):
    torch.manual_seed(0)
    x = (torch.randn(5, 5120, device="cuda") * 3).half()
    x[3] = 0
    xq, s = K.act_quant_int8(x)
    rq, rs = Q.quantize_activation_int8(x.cpu(), per_row=True)
    assert torch.allclose(s.cpu(), rs, rtol=1e-6, atol=0)
    assert torch.equal(xq.cpu(), rq)


@pytest.mark.parametrize("T", [1, 3, 8, 13, 32, 80])
@pytest.mark.parametrize("shape", [(5120, 1040), (17408, 520)])
def test_linear_w8a8(K, T, shape):
    Kd, N = shape
    g = torch.Generator().manual_seed(T)
    w = torch.randint(-128, 128, (N, Kd), generator=g, dtype=torch.int8)
    sw = torch.rand(N, generator=g) * 0.01 + 1e-3
    xq = torch.randint(-128, 128, (T, Kd), generator=g, dtype=torch.int8)
    sx = torch.rand(T, generator=g) * 0.05 + 1e-3
    ref = (xq.double() @ w.double().t()) * sx.double()[:, None] * sw.double()[None, :]
    out = K.linear_w8a8(w.cuda(), sw.cuda(), xq.cuda(), sx.cuda())
    assert torch.allclose(out.cpu().double(), ref, rtol=1e-5, atol=1e-5 * ref.abs().max().item())
    out16 = K.linear_w8a8(w.cuda(), sw.cuda(), xq.cuda(), sx.cuda(), out_dtype=torch.float16)
    assert torch.allclose(out16.cpu().double(), ref, rtol=2e-3, atol=2e-3 * ref.abs().max().item())


@pytest.mark.parametrize("T", [1, 8, 20, 70])
@pytest.mark.parametrize("group", [128, 256])
def test_linear_w4a8(K, T, group):
    Kd, N = 5120, 528
    lin = Q.random_int4_linear(Kd, N, group, generator=torch.Generator().manual_seed(T))
    wp, gs = Q.int4_to_w4a8(lin)
    g = torch.Generator().manual_seed(T + 1)
    xq = torch.randint(-128, 128, (T, Kd), generator=g, dtype=torch.int8)
    sx = torch.rand(T, generator=g) * 0.05 + 1e-3
    ref = (xq.double() @ Q.dequantize_w4a8(wp, gs, group).double().t()) * sx.double()[:, None]
    out = K.linear_w4a8(wp.cuda(), gs.cuda().contiguous(), xq.cuda(), sx.cuda(), group=group)
    assert torch.allclose(out.cpu().double(), ref, rtol=1e-4, atol=1e-5 * ref.abs().max().item())


def test_w8a8_end_to_end_close_to_fp16(K):
    """Quantise a real-valued layer and its input; the int8 product tracks the fp32 product."""
    torch.manual_seed(1)
    lin = Q.random_int4_linear(5120, 512, 128, generator=torch.Generator().manual_seed(3))
    w8, sw = Q.int4_to_w8a8(lin)
    x = torch.randn(4, 5120).half()
    xq, sx = K.act_quant_int8(x.cuda())
    out = K.linear_w8a8(w8.cuda(), sw.cuda(), xq, sx).cpu()
    ref = x.float() @ lin.dense().t()
    cos = torch.nn.functional.cosine_similarity(out.flatten(), ref.flatten(), dim=0)
    assert cos > 0.999
