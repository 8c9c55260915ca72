"""The INT8-activation FFN of one layer against the fp32 FFN of the same INT4 weights (reference test:
tests/test_engine_w8a8_w4a8.py compares its w8a8 / w4a8 engine output to w4a16 with loose bounds)."""
import pytest
import torch

from mi50grad_b200.utils import quant as Q

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["w8a8", "w4a8"])
@pytest.mark.parametrize("T", [1, 12])
def test_ffn_q8_tracks_w4a16(fmt, T):
    from mi50grad_b200.engine.ffn_q8 import FfnQ8, reference_ffn
    H, F = 256, 768
    g = torch.Generator().manual_seed(4)
    gate, up = Q.random_int4_linear(H, F, 128, generator=g), Q.random_int4_linear(H, F, 128, generator=g)
    down = Q.random_int4_linear(F, H, 128, generator=g)
    x = torch.randn(T, H, generator=g).half()
    ffn = FfnQ8(gate, up, down, fmt)
    out = ffn.forward(x.cuda()).cpu()
    ref = reference_ffn(gate, up, down, x)
    assert out.shape == ref.shape and torch.isfinite(out).all()
    cos = torch.nn.functional.cosine_similarity(out.flatten(), ref.flatten(), dim=0)
    assert cos > 0.995, float(cos)
    # the W4A8 weights are the INT4 weights themselves; W8A8 stores one byte per weight
    n_w = 2 * H * F + F * H
    assert ffn.weight_bytes() >= (n_w if fmt == "w8a8" else n_w // 2)
