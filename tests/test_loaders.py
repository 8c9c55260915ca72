import json

import pytest
import torch

from mi50grad_b200.config import load_config_from_json, tiny_config
from mi50grad_b200.loaders import (AWQWeightLoader, CompressedTensorsLoader, QwenWeightLoader,
                                   SafetensorsFile, detect_awq_format, detect_quant_format,
                                   load_any, load_awq_or_gptq, save_safetensors)
from mi50grad_b200.models.oracle import OracleEngine
from mi50grad_b200.models.weights import random_model, write_checkpoint
from mi50grad_b200.utils.quant import DenseLinear, Int4Linear


def _strip_zeros(mw):
    for lw in mw.layers:
        for lin in lw.linears().values():
            if isinstance(lin, Int4Linear):
                lin.zeros = None


def _hidden(mw, ids):
    e = OracleEngine(mw)
    return e.forward(e.embed(ids))


def test_safetensors_roundtrip(tmp_path):
    t = {"a": torch.arange(12, dtype=torch.int32).reshape(3, 4),
         "b": torch.randn(5).to(torch.bfloat16), "c": torch.randn(2, 2).half(),
         "e": torch.zeros(0, 3)}
    p = str(tmp_path / "x.safetensors")
    save_safetensors(p, t, {"k": "v"})
    f = SafetensorsFile(p)
    assert f.metadata == {"k": "v"}
    assert torch.equal(f.get("a"), t["a"])
    assert f.get("b").dtype == torch.bfloat16
    assert torch.equal(f.get("b", bf16_to=torch.float16), t["b"].half())
    assert f.get("e").shape == (0, 3)
    with pytest.raises(KeyError):
        f.get("zz")


@pytest.mark.parametrize("fmt,shards", [("gptq", 1), ("gptq", 3), ("awq", 1)])
def test_checkpoint_roundtrip_exact(tmp_path, fmt, shards):
    cfg = tiny_config()
    mw = random_model(cfg, 0)
    if fmt == "awq":
        _strip_zeros(mw)
    write_checkpoint(mw, str(tmp_path), fmt, shards=shards)
    assert detect_quant_format(str(tmp_path)) == fmt
    assert detect_awq_format(str(tmp_path)) == fmt
    cfg2 = load_config_from_json(str(tmp_path))
    assert cfg2.layer_types == cfg.layer_types and cfg2.head_dim == 64
    loader = load_awq_or_gptq(str(tmp_path), cfg2)
    assert isinstance(loader, AWQWeightLoader if fmt == "awq" else QwenWeightLoader)
    m2 = loader.load_model()
    ids = list(range(3, 15))
    assert torch.equal(_hidden(m2, ids), _hidden(mw, ids))
    assert loader.count_layers() == 4


def test_compressed_tensors_roundtrip(tmp_path):
    cfg = tiny_config(group_size=32)
    mw = random_model(cfg, 1)
    write_checkpoint(mw, str(tmp_path), "compressed-tensors")
    assert detect_quant_format(str(tmp_path)) == "compressed-tensors"
    cfg2 = load_config_from_json(str(tmp_path))
    assert cfg2.group_size == 32
    ld = CompressedTensorsLoader(str(tmp_path), cfg2)
    lw = ld.load_layer(3)
    # q_proj is de-interleaved along output features and keeps its scales
    assert isinstance(lw.q, Int4Linear) and lw.q.out_features == cfg.full_attn_q_dim
    assert torch.equal(lw.q.qweight, mw.layers[3].q.qweight)
    assert torch.equal(lw.q_gate.qweight, mw.layers[3].q_gate.qweight)
    # scales go through bf16 in this format
    assert torch.allclose(lw.q.scales.float(), mw.layers[3].q.scales.float(), rtol=1e-2)
    m2 = ld.load_model()
    ids = list(range(3, 15))
    a, b = _hidden(m2, ids), _hidden(mw, ids)
    assert (a - b).abs().max() / b.abs().max() < 6e-2


def test_fp16_attention_checkpoint_and_flag(tmp_path):
    cfg = tiny_config()
    mw = random_model(cfg, 2, int4_attention=False)
    write_checkpoint(mw, str(tmp_path), "gptq")
    cfg2 = load_config_from_json(str(tmp_path))
    assert cfg2.attn_quantized is False
    m2 = load_any(str(tmp_path)).load_model()
    assert isinstance(m2.layers[3].q, DenseLinear) and isinstance(m2.layers[3].gate, Int4Linear)
    assert isinstance(m2.layers[0].la_qkv, DenseLinear)
    ids = list(range(3, 15))
    assert torch.equal(_hidden(m2, ids), _hidden(mw, ids))


def test_norm_folding_and_tied_lm_head(tmp_path):
    cfg = tiny_config()
    mw = random_model(cfg, 3)
    mw.layers[0].attn_norm = torch.full_like(mw.layers[0].attn_norm, 1.5)
    write_checkpoint(mw, str(tmp_path), "gptq")
    ld = load_any(str(tmp_path))
    assert torch.allclose(ld.ck.get("model.language_model.layers.0.input_layernorm.weight").float(),
                          torch.full((256,), 0.5))
    assert torch.allclose(ld.load_layer(0).attn_norm.float(), torch.full((256,), 1.5))


def test_act_order_g_idx_falls_back_to_dense(tmp_path):
    cfg = tiny_config()
    mw = random_model(cfg, 4)
    write_checkpoint(mw, str(tmp_path), "gptq")
    from mi50grad_b200.loaders.safetensors_io import SafetensorsFile
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    T = {k: f.get(k) for k in f.keys()}
    key = "model.language_model.layers.0.mlp.gate_proj.g_idx"
    perm = torch.randperm(256, generator=torch.Generator().manual_seed(0))
    T[key] = (perm // 128).to(torch.int32)
    save_safetensors(str(tmp_path / "model.safetensors"), T)
    lw = load_any(str(tmp_path)).load_layer(0)
    assert isinstance(lw.gate, DenseLinear)
    from mi50grad_b200.utils.quant import unpack_int4_rows
    src = mw.layers[0].gate
    q = unpack_int4_rows(src.qweight).float()
    gi = T[key].long()
    exp = ((q - src.zeros.float()[gi]) * src.scales.float()[gi]).t()
    assert torch.allclose(lw.gate.weight.float(), exp, atol=2e-3)


def test_tp_sharded_load_matches_shard_of_full(tmp_path):
    cfg = tiny_config()
    mw = random_model(cfg, 5)
    write_checkpoint(mw, str(tmp_path), "gptq")
    ld = load_any(str(tmp_path))
    full = ld.load_layer(1)
    sh = ld.load_layer(1, tp_size=2, tp_rank=1)
    assert sh.down.group_offset == 352 % 128
    assert sh.gate.out_features == 352 and sh.down.in_features == 352
    assert torch.equal(sh.down.dense(), full.down.dense()[:, 352:])
    assert ld.load_lm_head(2, 1).shape == (512, 256)
    # the loader hands out views of the memory-mapped files: a rank's load materialises its shard only
    assert ld.ck.lazy and ld.ck.copied_bytes == 0
    qw = ld.ck.get("model.layers.1.mlp.down_proj.qweight" if "model.layers.1.mlp.down_proj.qweight" in ld.ck
                   else next(k for k in ld.ck.keys() if k.endswith("layers.1.mlp.down_proj.qweight")))
    # the row shard of down_proj is a window of the mapped file itself: no copy of the full tensor was made
    assert sh.down.qweight.untyped_storage().data_ptr() == qw.untyped_storage().data_ptr()
    assert sh.down.qweight.shape[0] * 2 == qw.shape[0]
