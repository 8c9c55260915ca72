"""Checkpoint loaders for the Qwen3.5 hybrid decoder: GPTQ-Int4, the
reference's zero-less "AWQ" variant, compressed-tensors pack-quantized, and
plain fp16/bf16 -- HuggingFace tensor names in, engine-format `LayerWeights` out.

One `CheckpointLoader` understands every format per projection (a projection is
INT4 when `<name>.qweight` or `<name>.weight_packed` exists, dense when
`<name>.weight` does), so mixed checkpoints -- INT4 FFN with fp16 attention,
which is what the reference actually ran (src/model/weight_loader.py:444-507) --
and fully quantised ones (its compressed-tensors path,
src/model/compressed_tensors_loader.py:382-518) go through the same code.  The
classes named like the reference's loaders are thin front-ends that pin the
format and keep the constructor signatures
(reference: src/model/weight_loader.py:390-413, src/model/awq_loader.py:124-154,
src/model/compressed_tensors_loader.py:189-236).

Differences from the reference, on purpose:
* `g_idx` is read.  A trivial map (k // group_size) is accepted silently; an
  act-order permutation cannot be expressed by group-contiguous kernels, so such
  a projection is dequantised to a dense fp16 matrix (the reference never reads
  g_idx at all).
* The compressed-tensors q_proj is de-interleaved along the output-feature axis
  and keeps its scales (the reference splits the wrong axis and drops scales:
  src/model/compressed_tensors_loader.py:412-472).
* True AutoAWQ tensors (N-packed qweight[K, N/8]) are recognised by shape and
  converted, not mis-read.
"""
from __future__ import annotations

import json
import logging
from pathlib import Path
from typing import Dict, List, Optional

import torch

from ..config import QwenConfig, load_config_from_json
from ..models.weights import LayerWeights, Linear, ModelWeights
from ..parallel.sharding import make_shard_spec, shard_layer
from ..utils.quant import (DenseLinear, Int4Linear, NIBBLES, autoawq_to_engine, ct_to_engine,
                           int4_to_w4a8, int4_to_w8a8, is_autoawq_layout, unpack_gptq_qzeros,
                           unpack_int4_rows)
from .safetensors_io import CheckpointDir

log = logging.getLogger(__name__)

LAYER_PREFIXES = ("model.language_model.layers.{i}", "model.layers.{i}",
                  "language_model.model.layers.{i}")
SKIP_PREFIXES = ("model.visual.", "model.merger.", "mtp.")


def detect_awq_format(model_dir: str) -> str:
    """'awq' when INT4 projections carry qweight+scales but no qzeros, 'gptq'
    when qzeros exist, else 'unknown' (reference: src/model/awq_loader.py:38-85)."""
    ck = CheckpointDir(model_dir)
    keys = ck.keys()
    ck.close()
    has_q = any(k.endswith(".qweight") for k in keys)
    has_z = any(k.endswith(".qzeros") for k in keys)
    if has_q and not has_z:
        return "awq"
    if has_q:
        return "gptq"
    return "unknown"


def detect_compressed_tensors_format(model_dir: str) -> bool:
    cfgp = Path(model_dir) / "config.json"
    if cfgp.exists():
        hf = json.loads(cfgp.read_text())
        q = hf.get("quantization_config", hf.get("text_config", {}).get("quantization_config", {})) or {}
        if q.get("quant_method") == "compressed-tensors":
            return True
    ck = CheckpointDir(model_dir)
    found = any(k.endswith(".weight_packed") for k in ck.keys())
    ck.close()
    return found


def detect_quant_format(model_dir: str) -> str:
    """-> 'compressed-tensors' | 'awq' | 'gptq' | 'fp16'
    (reference: src/model/compressed_tensors_loader.py:80-95)."""
    if detect_compressed_tensors_format(model_dir):
        return "compressed-tensors"
    f = detect_awq_format(model_dir)
    return f if f in ("awq", "gptq") else "fp16"


class CheckpointLoader:
    def __init__(self, model_dir: str, config: Optional[QwenConfig] = None,
                 group_size: Optional[int] = None, quant_format: str = "w4a16",
                 fmt: Optional[str] = None):
        self.model_dir = str(model_dir)
        self.fmt = fmt or detect_quant_format(model_dir)
        if config is None:
            config = load_config_from_json(model_dir)
            group_size = group_size or config.group_size
        self.config = config
        self.group_size = group_size or (32 if self.fmt == "compressed-tensors"
                                         else self.config.group_size)
        self.quant_format = quant_format
        # tensors are views of the memory-mapped files: a tensor-parallel rank slices its shard out of them
        # and only those pages are ever read (the reference reads every full tensor on every GPU's behalf:
        # src/model/weight_loader.py:300-316)
        self.ck = CheckpointDir(model_dir, SKIP_PREFIXES, lazy=True)
        self.layer_prefix = self._detect_layer_prefix()
        self.model_prefix = self.layer_prefix.rsplit(".layers.", 1)[0]

    def _detect_layer_prefix(self) -> str:
        for p in LAYER_PREFIXES:
            if f"{p.format(i=0)}.input_layernorm.weight" in self.ck:
                return p
        raise FileNotFoundError("no decoder layer tensors found under any known prefix")

    # -- tensors --------------------------------------------------------------
    def load_tensor(self, key: str) -> torch.Tensor:
        return self.ck.get(key)

    def load_linear(self, name: str) -> Linear:
        ck = self.ck
        if f"{name}.weight_packed" in ck:
            packed, scale = ck.get(f"{name}.weight_packed"), ck.get(f"{name}.weight_scale")
            K, G = packed.shape[1] * NIBBLES, scale.shape[1]
            g = K // G if K % G == 0 else self.group_size
            return ct_to_engine(packed, scale, g)
        if f"{name}.qweight" in ck:
            qw, sc = ck.get(f"{name}.qweight"), ck.get(f"{name}.scales").to(torch.float16)
            if is_autoawq_layout(qw.shape, sc.shape):
                if f"{name}.qzeros" not in ck:
                    raise ValueError(f"{name}: AutoAWQ-layout qweight without qzeros")
                return autoawq_to_engine(qw, ck.get(f"{name}.qzeros"), sc, self.group_size)
            zeros = None
            if f"{name}.qzeros" in ck:
                zeros = unpack_gptq_qzeros(ck.get(f"{name}.qzeros"), sym=self.config.quant_sym)
            lin = Int4Linear(qw, sc, zeros, self.group_size, 0)
            lin.validate()
            if f"{name}.g_idx" in ck:
                g_idx = ck.get(f"{name}.g_idx").to(torch.int64)
                trivial = torch.arange(lin.in_features) // self.group_size
                if not torch.equal(g_idx, trivial):
                    log.warning("%s uses act-order (non-trivial g_idx): dequantising to fp16", name)
                    q = unpack_int4_rows(qw).float()
                    z = 0.0 if zeros is None else zeros.float()[g_idx]
                    return DenseLinear(((q - z) * sc.float()[g_idx]).t().contiguous().half())
            return lin
        if f"{name}.weight" in ck:
            return DenseLinear(ck.get(f"{name}.weight").to(torch.float16))
        raise FileNotFoundError(f"Cannot find tensor: {name}.(weight|qweight|weight_packed)")

    def _norm(self, key: str) -> torch.Tensor:
        return (1.0 + self.ck.get(key).float()).to(torch.float16)

    @staticmethod
    def _split_q_gate(lin: Linear, heads: int, hd: int):
        """HF q_proj output features are per head [Q_h | gate_h]."""
        if isinstance(lin, DenseLinear):
            w = lin.weight.reshape(heads, 2 * hd, -1)
            return (DenseLinear(w[:, :hd].reshape(heads * hd, -1).contiguous()),
                    DenseLinear(w[:, hd:].reshape(heads * hd, -1).contiguous()))
        idx = torch.arange(heads * 2 * hd).reshape(heads, 2, hd)
        qi, gi = idx[:, 0].reshape(-1), idx[:, 1].reshape(-1)
        pick = lambda t, i: None if t is None else t[:, i].contiguous()
        mk = lambda i: Int4Linear(pick(lin.qweight, i), pick(lin.scales, i), pick(lin.zeros, i),
                                  lin.group_size, lin.group_offset)
        return mk(qi), mk(gi)

    # -- layers ---------------------------------------------------------------
    def load_layer(self, layer_idx: int, tp_size: int = 1, tp_rank: int = 0) -> LayerWeights:
        cfg = self.config
        p = self.layer_prefix.format(i=layer_idx)
        lw = LayerWeights(
            layer_type=cfg.layer_types[layer_idx],
            attn_norm=self._norm(f"{p}.input_layernorm.weight"),
            ffn_norm=self._norm(f"{p}.post_attention_layernorm.weight"),
            gate=self.load_linear(f"{p}.mlp.gate_proj"),
            up=self.load_linear(f"{p}.mlp.up_proj"),
            down=self.load_linear(f"{p}.mlp.down_proj"))
        if lw.is_full:
            a = f"{p}.self_attn"
            lw.q, lw.q_gate = self._split_q_gate(self.load_linear(f"{a}.q_proj"),
                                                 cfg.num_attention_heads, cfg.head_dim)
            lw.k = self.load_linear(f"{a}.k_proj")
            lw.v = self.load_linear(f"{a}.v_proj")
            lw.o = self.load_linear(f"{a}.o_proj")
            lw.q_norm = self._norm(f"{a}.q_norm.weight")
            lw.k_norm = self._norm(f"{a}.k_norm.weight")
        else:
            la = f"{p}.linear_attn"
            lw.la_qkv = self.load_linear(f"{la}.in_proj_qkv")
            lw.la_a = self.load_linear(f"{la}.in_proj_a")
            lw.la_b = self.load_linear(f"{la}.in_proj_b")
            lw.la_z = self.load_linear(f"{la}.in_proj_z")
            lw.la_out = self.load_linear(f"{la}.out_proj")
            conv = self.ck.get(f"{la}.conv1d.weight").to(torch.float16)
            lw.la_conv1d = conv.reshape(conv.shape[0], -1).contiguous()
            lw.la_A_log = self.ck.get(f"{la}.A_log").float()
            lw.la_dt_bias = self.ck.get(f"{la}.dt_bias").to(torch.float16)
            lw.la_norm = self.ck.get(f"{la}.norm.weight").to(torch.float16)
        return shard_layer(lw, cfg, tp_size, tp_rank)

    def load_layer_alt_format(self, layer_idx: int) -> Dict[str, torch.Tensor]:
        """FFN weights in the W8A8 / W4A8 forms (reference:
        src/model/weight_loader.py:520-537)."""
        lw = self.load_layer(layer_idx)
        out: Dict[str, torch.Tensor] = {}
        for n in ("gate", "up", "down"):
            lin = getattr(lw, n)
            if not isinstance(lin, Int4Linear):
                continue
            if self.quant_format == "w8a8":
                out[f"{n}_w8a8"], out[f"{n}_scale_w8a8"] = int4_to_w8a8(lin)
            elif self.quant_format == "w4a8":
                out[f"{n}_w4a8"], out[f"{n}_scale_w4a8"] = int4_to_w4a8(lin)
        return out

    def load_embedding(self) -> torch.Tensor:
        return self.ck.get(f"{self.model_prefix}.embed_tokens.weight").to(torch.float16)

    def load_lm_head(self, tp_size: int = 1, tp_rank: int = 0) -> torch.Tensor:
        """Falls back to the tied embedding (reference: src/model/weight_loader.py:545-551)."""
        w = self.ck.get("lm_head.weight") if "lm_head.weight" in self.ck else self.load_embedding()
        w = w.to(torch.float16)
        if tp_size > 1:
            a, b = make_shard_spec(self.config, tp_size, tp_rank).vocab
            w = w[a:b].contiguous()
        return w

    def load_final_norm(self) -> torch.Tensor:
        return self._norm(f"{self.model_prefix}.norm.weight")

    def load_model(self, tp_size: int = 1, tp_rank: int = 0) -> ModelWeights:
        mw = ModelWeights(self.config)
        mw.layers = [self.load_layer(i, tp_size, tp_rank)
                     for i in range(self.config.num_hidden_layers)]
        mw.embed = self.load_embedding()
        mw.lm_head = self.load_lm_head(tp_size, tp_rank)
        mw.final_norm = self.load_final_norm()
        return mw

    def get_all_tensor_keys(self) -> List[str]:
        return self.ck.keys()

    def count_layers(self) -> int:
        n = 0
        while f"{self.layer_prefix.format(i=n)}.input_layernorm.weight" in self.ck:
            n += 1
        return n


class QwenWeightLoader(CheckpointLoader):
    """GPTQ front-end (reference: src/model/weight_loader.py:390-413)."""

    def __init__(self, model_dir: str, config: QwenConfig, bits: int = 4,
                 group_size: int = 128, quant_format: str = "w4a16"):
        if bits != 4:
            raise ValueError("only 4-bit weights are supported")
        super().__init__(model_dir, config, group_size, quant_format, fmt="gptq")


class AWQWeightLoader(CheckpointLoader):
    """The reference's AWQ definition: GPTQ tensors without qzeros, w = q*scale
    (reference: src/model/awq_loader.py:124-154)."""

    def __init__(self, model_dir: str, config: QwenConfig, group_size: int = 128):
        super().__init__(model_dir, config, group_size, fmt="awq")


class CompressedTensorsLoader(CheckpointLoader):
    """compressed-tensors pack-quantized, group 32, symmetric
    (reference: src/model/compressed_tensors_loader.py:189-236)."""

    def __init__(self, model_dir: str, config: QwenConfig, group_size: int = 32):
        super().__init__(model_dir, config, group_size, fmt="compressed-tensors")


def awq_dequantize(qweight: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """-> W[K, N] fp32 = q * scale (reference: src/model/awq_loader.py:88-121)."""
    return Int4Linear(qweight, scales, None, group_size).dense().t().contiguous()


def load_awq_or_gptq(model_dir: str, config: QwenConfig, fmt: str = "auto") -> CheckpointLoader:
    """(reference: src/model/awq_loader.py:399-420)"""
    if fmt == "auto":
        fmt = detect_awq_format(model_dir)
    if fmt == "awq":
        return AWQWeightLoader(model_dir, config, config.group_size)
    return QwenWeightLoader(model_dir, config, config.bits, config.group_size)


def load_compressed_tensors(model_dir: str, config: QwenConfig, group_size: int = 32):
    return CompressedTensorsLoader(model_dir, config, group_size)


def load_any(model_dir: str, config: Optional[QwenConfig] = None) -> CheckpointLoader:
    return CheckpointLoader(model_dir, config)
