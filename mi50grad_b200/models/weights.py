"""Engine-format weights of the hybrid decoder, random initialisation, and a
writer that emits HuggingFace-named GPTQ / AWQ / compressed-tensors checkpoints
(used by the loader tests the way the reference's tests build synthetic
safetensors: tests/test_awq_loader.py:38-45).

A `LayerWeights` holds one decoder layer in the form the engines consume
(reference: src/inference/engine.py:372-455 keeps a bag of device pointers; here
each projection is a `DenseLinear` or `Int4Linear` object that the sharder, the
CPU oracle and the CUDA uploader all understand).  Norm vectors are *effective*
multipliers: the `1 + w` of Qwen's RMSNorm is folded in when a checkpoint is
read (reference: src/model/weight_loader.py:439-440), the DeltaNet output norm
is used as stored (reference: src/model/weight_loader.py:506).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Union

import torch

from ..config import QwenConfig
from ..utils.quant import (DenseLinear, Int4Linear, engine_to_ct, pack_gptq_qzeros,
                           random_int4_linear)

Linear = Union[DenseLinear, Int4Linear]

FULL_LINEARS = ("q", "q_gate", "k", "v", "o")
LA_LINEARS = ("la_qkv", "la_a", "la_b", "la_z", "la_out")
FFN_LINEARS = ("gate", "up", "down")


@dataclass
class LayerWeights:
    layer_type: str
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor
    gate: Linear = None
    up: Linear = None
    down: Linear = None
    # gated full attention
    q: Optional[Linear] = None
    q_gate: Optional[Linear] = None
    k: Optional[Linear] = None
    v: Optional[Linear] = None
    o: Optional[Linear] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    # Gated DeltaNet
    la_qkv: Optional[Linear] = None
    la_a: Optional[Linear] = None
    la_b: Optional[Linear] = None
    la_z: Optional[Linear] = None
    la_out: Optional[Linear] = None
    la_conv1d: Optional[torch.Tensor] = None     # [conv_dim, kernel]
    la_A_log: Optional[torch.Tensor] = None      # [v_heads] fp32
    la_dt_bias: Optional[torch.Tensor] = None    # [v_heads]
    la_norm: Optional[torch.Tensor] = None       # [v_head_dim]

    @property
    def is_full(self) -> bool:
        return self.layer_type == "full_attention"

    def linears(self) -> Dict[str, Linear]:
        names = (FULL_LINEARS if self.is_full else LA_LINEARS) + FFN_LINEARS
        return {n: getattr(self, n) for n in names}


@dataclass
class ModelWeights:
    config: QwenConfig
    layers: List[LayerWeights] = field(default_factory=list)
    embed: Optional[torch.Tensor] = None        # [vocab, hidden] fp16
    lm_head: Optional[torch.Tensor] = None      # [vocab, hidden] fp16
    final_norm: Optional[torch.Tensor] = None   # [hidden]


def _dense(N, K, gen, device, std=0.02):
    return DenseLinear((torch.randn(N, K, generator=gen, device=device) * std).to(torch.float16))


def _proj(N, K, int4, cfg, gen, device) -> Linear:
    if int4:
        return random_int4_linear(K, N, cfg.group_size, gen, device)
    return _dense(N, K, gen, device)


def random_layer(cfg: QwenConfig, layer_idx: int, gen: torch.Generator, device="cpu",
                 int4_attention: bool = True) -> LayerWeights:
    """Random weights of the benchmark's form: INT4 (nibbles uniform, zero 8,
    scales U(0.002, 0.02)) for every large projection, fp16 for the small DeltaNet
    tensors, all norm multipliers equal to one."""
    h, inter = cfg.hidden_size, cfg.intermediate_size
    ones = lambda n: torch.ones(n, dtype=torch.float16, device=device)
    lw = LayerWeights(
        layer_type=cfg.layer_types[layer_idx], attn_norm=ones(h), ffn_norm=ones(h),
        gate=random_int4_linear(h, inter, cfg.group_size, gen, device),
        up=random_int4_linear(h, inter, cfg.group_size, gen, device),
        down=random_int4_linear(inter, h, cfg.group_size, gen, device),
    )
    if lw.is_full:
        qd, kvd = cfg.full_attn_q_dim, cfg.full_attn_kv_dim
        lw.q = _proj(qd, h, int4_attention, cfg, gen, device)
        lw.q_gate = _proj(qd, h, int4_attention, cfg, gen, device)
        lw.k = _proj(kvd, h, int4_attention, cfg, gen, device)
        lw.v = _proj(kvd, h, int4_attention, cfg, gen, device)
        lw.o = _proj(h, qd, int4_attention, cfg, gen, device)
        lw.q_norm = ones(cfg.head_dim)
        lw.k_norm = ones(cfg.head_dim)
    else:
        nv, vd = cfg.linear_num_value_heads, cfg.linear_attn_value_dim
        lw.la_qkv = _proj(cfg.linear_conv_dim, h, int4_attention, cfg, gen, device)
        lw.la_z = _proj(vd, h, int4_attention, cfg, gen, device)
        lw.la_a = _dense(nv, h, gen, device)
        lw.la_b = _dense(nv, h, gen, device)
        lw.la_out = _proj(h, vd, int4_attention, cfg, gen, device)
        lw.la_conv1d = (torch.randn(cfg.linear_conv_dim, cfg.linear_conv_kernel_dim,
                                    generator=gen, device=device) * 0.3).to(torch.float16)
        lw.la_A_log = (torch.rand(nv, generator=gen, device=device) * 1.5 - 1.0).float()
        lw.la_dt_bias = (torch.randn(nv, generator=gen, device=device) * 0.5).to(torch.float16)
        lw.la_norm = ones(cfg.linear_value_head_dim)
    return lw


def random_model(cfg: QwenConfig, seed: int = 0, device="cpu", int4_attention: bool = True,
                 embed_std: float = 0.05) -> ModelWeights:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    mw = ModelWeights(cfg)
    for i in range(cfg.num_hidden_layers):
        mw.layers.append(random_layer(cfg, i, gen, device, int4_attention))
    h, v = cfg.hidden_size, cfg.vocab_size
    mw.embed = (torch.randn(v, h, generator=gen, device=device) * embed_std).to(torch.float16)
    mw.lm_head = (torch.randn(v, h, generator=gen, device=device) * embed_std).to(torch.float16)
    mw.final_norm = torch.ones(h, dtype=torch.float16, device=device)
    return mw


# ---------------------------------------------------------------------------
# Checkpoint writer (HuggingFace tensor names).
# ---------------------------------------------------------------------------

def _interleave_q_gate(q: torch.Tensor, g: torch.Tensor, heads: int, hd: int) -> torch.Tensor:
    """HF q_proj rows are per head [Q_h(hd), gate_h(hd)] (reference:
    src/model/weight_loader.py:463-471).  Works on dim 0."""
    rest = q.shape[1:]
    return torch.stack([q.reshape(heads, hd, *rest), g.reshape(heads, hd, *rest)], dim=1) \
        .reshape(2 * heads * hd, *rest)


def _interleave_cols(a: torch.Tensor, b: torch.Tensor, heads: int, hd: int) -> torch.Tensor:
    """Same interleave along the last dim of a [R, heads*hd] tensor."""
    return _interleave_q_gate(a.t().contiguous(), b.t().contiguous(), heads, hd).t().contiguous()


def _emit_linear(out: Dict[str, torch.Tensor], name: str, lin: Linear, fmt: str, sym=True):
    if isinstance(lin, DenseLinear):
        out[f"{name}.weight"] = lin.weight
        return
    if fmt == "compressed-tensors":
        packed, scale = engine_to_ct(lin)
        out[f"{name}.weight_packed"] = packed
        out[f"{name}.weight_scale"] = scale.to(torch.bfloat16)
        out[f"{name}.weight_shape"] = torch.tensor([lin.out_features, lin.in_features],
                                                   dtype=torch.int64)
        return
    out[f"{name}.qweight"] = lin.qweight
    out[f"{name}.scales"] = lin.scales
    if fmt == "gptq":
        zeros = lin.zeros if lin.zeros is not None else torch.zeros_like(lin.scales)
        out[f"{name}.qzeros"] = pack_gptq_qzeros(zeros, sym=sym)
        K = lin.in_features
        out[f"{name}.g_idx"] = (torch.arange(K) // lin.group_size).to(torch.int32)


def _cat_int4_cols(a: Int4Linear, b: Int4Linear, heads: int, hd: int) -> Int4Linear:
    z = None if a.zeros is None else _interleave_cols(a.zeros, b.zeros, heads, hd)
    return Int4Linear(_interleave_cols(a.qweight, b.qweight, heads, hd),
                      _interleave_cols(a.scales, b.scales, heads, hd), z,
                      a.group_size, a.group_offset)


def write_checkpoint(mw: ModelWeights, out_dir: str, fmt: str = "gptq",
                     prefix: str = "model.language_model", shards: int = 1) -> None:
    """Write `mw` as a HuggingFace-style directory (config.json + safetensors).
    fmt is 'gptq', 'awq' (the reference's zero-less GPTQ variant) or
    'compressed-tensors'.  Norms are written as `w - 1` so that a loader that
    folds `1 + w` recovers them."""
    from ..loaders.safetensors_io import save_safetensors
    cfg = mw.config
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    T: Dict[str, torch.Tensor] = {}
    unfold = lambda w: (w.float() - 1.0).to(torch.float16)
    for i, lw in enumerate(mw.layers):
        p = f"{prefix}.layers.{i}"
        T[f"{p}.input_layernorm.weight"] = unfold(lw.attn_norm)
        T[f"{p}.post_attention_layernorm.weight"] = unfold(lw.ffn_norm)
        if lw.is_full:
            nh, hd = cfg.num_attention_heads, cfg.head_dim
            if isinstance(lw.q, DenseLinear):
                qcat: Linear = DenseLinear(_interleave_q_gate(lw.q.weight, lw.q_gate.weight, nh, hd))
            else:
                qcat = _cat_int4_cols(lw.q, lw.q_gate, nh, hd)
            _emit_linear(T, f"{p}.self_attn.q_proj", qcat, fmt)
            _emit_linear(T, f"{p}.self_attn.k_proj", lw.k, fmt)
            _emit_linear(T, f"{p}.self_attn.v_proj", lw.v, fmt)
            _emit_linear(T, f"{p}.self_attn.o_proj", lw.o, fmt)
            T[f"{p}.self_attn.q_norm.weight"] = unfold(lw.q_norm)
            T[f"{p}.self_attn.k_norm.weight"] = unfold(lw.k_norm)
        else:
            la = f"{p}.linear_attn"
            _emit_linear(T, f"{la}.in_proj_qkv", lw.la_qkv, fmt)
            _emit_linear(T, f"{la}.in_proj_a", lw.la_a, fmt)
            _emit_linear(T, f"{la}.in_proj_b", lw.la_b, fmt)
            _emit_linear(T, f"{la}.in_proj_z", lw.la_z, fmt)
            _emit_linear(T, f"{la}.out_proj", lw.la_out, fmt)
            T[f"{la}.conv1d.weight"] = lw.la_conv1d.unsqueeze(1)
            T[f"{la}.A_log"] = lw.la_A_log.float()
            T[f"{la}.dt_bias"] = lw.la_dt_bias
            T[f"{la}.norm.weight"] = lw.la_norm.float()
        for n in FFN_LINEARS:
            _emit_linear(T, f"{p}.mlp.{n}_proj", getattr(lw, n), fmt)
    T[f"{prefix}.embed_tokens.weight"] = mw.embed
    T["lm_head.weight"] = mw.lm_head
    T[f"{prefix}.norm.weight"] = unfold(mw.final_norm)

    names = list(T)
    per = -(-len(names) // shards)
    weight_map = {}
    for s in range(shards):
        fn = "model.safetensors" if shards == 1 else f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        part = {k: T[k] for k in names[s * per:(s + 1) * per]}
        save_safetensors(str(out_dir / fn), part)
        weight_map.update({k: fn for k in part})
    if shards > 1:
        (out_dir / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))

    attn_int4 = any(isinstance(l, Int4Linear) for lw in mw.layers
                    for n, l in lw.linears().items() if n not in FFN_LINEARS)
    if fmt == "compressed-tensors":
        g = next(l.group_size for lw in mw.layers for l in lw.linears().values()
                 if isinstance(l, Int4Linear))
        qc = {"quant_method": "compressed-tensors", "format": "pack-quantized",
              "config_groups": {"group_0": {"weights": {"num_bits": 4, "group_size": g,
                                                        "symmetric": True, "type": "int"}}}}
    else:
        qc = {"quant_method": fmt, "bits": 4, "group_size": cfg.group_size, "sym": True}
        if not attn_int4:
            qc["dynamic"] = {"-:.*attn.*": {}}
    text = {k: getattr(cfg, k) for k in (
        "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
        "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings",
        "rms_norm_eps", "full_attention_interval", "layer_types", "linear_key_head_dim",
        "linear_num_key_heads", "linear_num_value_heads", "linear_value_head_dim",
        "linear_conv_kernel_dim", "attn_output_gate", "rope_style")}
    text["rope_parameters"] = {"rope_theta": cfg.rope_theta,
                               "partial_rotary_factor": cfg.partial_rotary_factor,
                               "mrope_section": cfg.mrope_sections,
                               "mrope_interleaved": cfg.mrope_interleaved}
    (out_dir / "config.json").write_text(json.dumps(
        {"text_config": text, "quantization_config": qc}, indent=1))
