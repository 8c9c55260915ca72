import torch
import pytest

from mi50grad_b200.utils import quant as Q


def test_pack_roundtrip_rows_and_cols():
    g = torch.Generator().manual_seed(0)
    q = torch.randint(0, 16, (64, 24), generator=g, dtype=torch.uint8)
    assert torch.equal(Q.unpack_int4_rows(Q.pack_int4_rows(q)), q)
    assert torch.equal(Q.unpack_int4_cols(Q.pack_int4_cols(q)), q)
    w = Q.pack_int4_rows(q)
    assert w.dtype == torch.int32 and w.shape == (8, 24)
    # nibble b of word r holds k = 8r + b
    assert int(w[1, 3].item()) & 0xF == int(q[8, 3])
    assert (int(w[1, 3].item()) >> 28) & 0xF == int(q[15, 3])


def test_qzeros_sym_and_asym():
    z = torch.full((3, 16), 8.0)
    assert torch.equal(Q.unpack_gptq_qzeros(Q.pack_gptq_qzeros(z, sym=True), sym=True), z.half())
    z2 = torch.randint(1, 16, (3, 16)).float()
    assert torch.equal(Q.unpack_gptq_qzeros(Q.pack_gptq_qzeros(z2, sym=False), sym=False), z2.half())


@pytest.mark.parametrize("sym", [True, False])
def test_quantize_dequantize_error(sym):
    g = torch.Generator().manual_seed(1)
    w = torch.randn(48, 320, generator=g) * 0.05
    lin = Q.quantize_int4(w, 128, sym=sym)
    lin.validate()
    err = (lin.dense() - w).abs().max()
    assert err < 0.05 * 4 / 7 + 1e-3


def test_short_last_group_and_offset_dense():
    g = torch.Generator().manual_seed(2)
    lin = Q.random_int4_linear(704, 40, 128, g)
    assert lin.num_groups == 6
    full = lin.dense()
    from mi50grad_b200.parallel.sharding import slice_in
    a, b = slice_in(lin, 0, 352), slice_in(lin, 352, 704)
    assert b.group_offset == 352 % 128 and b.num_groups == 4 and a.num_groups == 3
    a.validate(); b.validate()
    assert torch.equal(torch.cat([a.dense(), b.dense()], dim=1), full)


def test_awq_form_has_no_zero():
    g = torch.Generator().manual_seed(3)
    lin = Q.random_int4_linear(256, 8, 128, g, zeros=None)
    q = Q.unpack_int4_rows(lin.qweight).float()
    exp = (q * lin.scales.float().repeat_interleave(128, 0)).t()
    assert torch.allclose(lin.dense(), exp)


def test_ct_roundtrip():
    g = torch.Generator().manual_seed(4)
    lin = Q.random_int4_linear(128, 16, 32, g)
    packed, scale = Q.engine_to_ct(lin)
    assert packed.shape == (16, 16) and scale.shape == (16, 4)
    back = Q.ct_to_engine(packed, scale, 32)
    assert torch.equal(back.qweight, lin.qweight)
    assert torch.allclose(back.dense(), lin.dense())


def test_autoawq_layout_detected_and_converted():
    g = torch.Generator().manual_seed(5)
    K, N = 256, 32
    q = torch.randint(0, 16, (K, N), generator=g, dtype=torch.uint8)
    z = torch.randint(0, 16, (2, N), generator=g, dtype=torch.uint8)
    s = (torch.rand(2, N, generator=g) * 0.01 + 0.001).half()

    def pack_awq(x):
        out = torch.zeros(x.shape[0], x.shape[1] // 8, dtype=torch.int64)
        for slot, col in enumerate(Q.AUTOAWQ_ORDER):
            out |= x[:, col::8].to(torch.int64) << (4 * slot)
        return Q._to_i32(out)
    qw, qz = pack_awq(q), pack_awq(z)
    assert Q.is_autoawq_layout(qw.shape, s.shape)
    assert not Q.is_autoawq_layout((K // 8, N), s.shape)
    lin = Q.autoawq_to_engine(qw, qz, s, 128)
    exp = ((q.float() - z.float().repeat_interleave(128, 0)) * s.float().repeat_interleave(128, 0)).t()
    assert torch.allclose(lin.dense(), exp)


def test_w8a8_and_w4a8_conversions():
    g = torch.Generator().manual_seed(6)
    lin = Q.random_int4_linear(256, 24, 128, g)
    w = lin.dense()
    w8, s8 = Q.int4_to_w8a8(lin)
    assert w8.dtype == torch.int8 and w8.shape == (24, 256)
    assert (w8.float() * s8[:, None] - w).abs().max() <= s8.max() * 0.51
    w4, s4 = Q.int4_to_w4a8(lin)
    assert w4.shape == (24, 32)
    assert torch.allclose(Q.dequantize_w4a8(w4, s4, 128), w, atol=1e-6)
    x = torch.randn(256, generator=g)
    xq, sx = Q.quantize_activation_int8(x)
    assert (xq.float() * sx - x).abs().max() <= sx * 0.51


def test_ffn_q8_rejects_unknown_format_and_reference_shape():
    from mi50grad_b200.engine.ffn_q8 import FfnQ8, reference_ffn
    g = torch.Generator().manual_seed(0)
    gate, up = Q.random_int4_linear(128, 256, 128, generator=g), Q.random_int4_linear(128, 256, 128, generator=g)
    down = Q.random_int4_linear(256, 128, 128, generator=g)
    with pytest.raises(ValueError):
        FfnQ8(gate, up, down, "w2a2", device="cpu")
    assert reference_ffn(gate, up, down, torch.randn(3, 128)).shape == (3, 128)
    ffn = FfnQ8(gate, up, down, "w4a8", device="cpu")             # conversion and storage need no GPU
    assert ffn.weight_bytes() == 3 * (128 * 256 // 2) + 2 * (1 * 256 * 2) + 2 * 128 * 2


def test_w4a8_per_channel_and_dense_roundtrip():
    g = torch.Generator().manual_seed(2)
    lin = Q.random_int4_linear(256, 64, 128, generator=g)
    packed, s_ch = Q.int4_to_w4a8_per_channel(lin)
    p2, s_grp = Q.int4_to_w4a8(lin)
    assert torch.equal(packed, p2) and s_ch.shape == (64,)
    assert torch.allclose(s_ch, s_grp.float().mean(dim=0))
    w = torch.randn(48, 256, generator=g)
    assert Q.w4a8_roundtrip_error(w, 128) < 0.5 / 7 + 1e-3          # half a step of a 4-bit symmetric grid
    pk, sc = Q.dense_to_w4a8(w, 128)
    assert pk.shape == (48, 32) and pk.dtype == torch.int32 and sc.shape == (2, 48) and sc.dtype == torch.float16
