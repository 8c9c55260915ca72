"""Model and engine configuration.

`QwenConfig` carries every dimension of the Qwen3.5 hybrid decoder (Gated
DeltaNet + gated full attention) with the same field names and defaults as the
reference's dataclass (reference: src/model/qwen.py:26-115), plus the JSON
loader for HuggingFace `config.json` files (reference: src/model/qwen.py:140-192)
and the memory estimators (reference: src/model/qwen.py:195-253), re-sized for a
180 GB B200 instead of a 16/32 GB MI50.

`EngineConfig` replaces the reference's ~20 imperative `set_*` toggles
(reference: src/inference/tp_engine.py:2252-2527) with one frozen description
of how the engine runs; the `set_*` names survive as thin shims on the engines.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import List, Optional

B200_HBM_BYTES = 180 * 10**9


@dataclass
class QwenConfig:
    hidden_size: int = 5120
    intermediate_size: int = 17408
    num_hidden_layers: int = 64
    num_attention_heads: int = 24
    num_key_value_heads: int = 4
    head_dim: int = 256
    vocab_size: int = 248320
    max_position_embeddings: int = 262144
    rope_theta: float = 10000000.0
    rms_norm_eps: float = 1e-6

    full_attention_interval: int = 4
    layer_types: List[str] = field(default_factory=list)

    linear_key_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 48
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4

    partial_rotary_factor: float = 0.25
    mrope_sections: List[int] = field(default_factory=lambda: [11, 11, 10])
    mrope_interleaved: bool = True
    # 'interleaved' rotates pairs (2i, 2i+1) as the reference kernels do
    # (reference: src/kernels/qknorm_rope.hip:140-152); 'half' rotates
    # (i, i + rot/2) like HuggingFace's rotate_half.
    rope_style: str = "interleaved"

    quant_method: str = "gptq"
    bits: int = 4
    group_size: int = 128
    quant_sym: bool = True
    attn_quantized: bool = False

    attn_output_gate: bool = True

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = [
                "full_attention" if (i + 1) % self.full_attention_interval == 0
                else "linear_attention"
                for i in range(self.num_hidden_layers)
            ]
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types length must equal num_hidden_layers")

    # -- layer kinds -----------------------------------------------------
    def is_full_attention(self, layer_idx: int) -> bool:
        return self.layer_types[layer_idx] == "full_attention"

    def is_linear_attention(self, layer_idx: int) -> bool:
        return self.layer_types[layer_idx] == "linear_attention"

    @property
    def num_full_attention_layers(self) -> int:
        return sum(t == "full_attention" for t in self.layer_types)

    @property
    def num_linear_attention_layers(self) -> int:
        return sum(t == "linear_attention" for t in self.layer_types)

    # -- derived dims ------------------------------------------------------
    @property
    def full_attn_q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def full_attn_kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def linear_attn_key_dim(self) -> int:
        return self.linear_num_key_heads * self.linear_key_head_dim

    @property
    def linear_attn_value_dim(self) -> int:
        return self.linear_num_value_heads * self.linear_value_head_dim

    @property
    def linear_conv_dim(self) -> int:
        return 2 * self.linear_attn_key_dim + self.linear_attn_value_dim

    @property
    def kv_heads_per_group(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    def full_attention_layer_indices(self) -> List[int]:
        return [i for i, t in enumerate(self.layer_types) if t == "full_attention"]

    def linear_attention_layer_indices(self) -> List[int]:
        return [i for i, t in enumerate(self.layer_types) if t == "linear_attention"]

    def max_tp(self) -> int:
        """Largest tensor-parallel degree the head counts allow.  KV heads are
        replicated when tp > num_key_value_heads, so the bound comes from the
        query heads, the DeltaNet key heads and the FFN width."""
        tp = 1
        while True:
            nxt = tp * 2
            if (self.num_attention_heads % nxt or self.linear_num_key_heads % nxt
                    or self.linear_num_value_heads % nxt
                    or self.intermediate_size % (8 * nxt)):
                return tp
            tp = nxt


def qwen35_27b(**overrides) -> QwenConfig:
    """The Qwen3.5-27B architecture the headline benchmark names."""
    return QwenConfig(**overrides)


def tiny_config(**overrides) -> QwenConfig:
    """The 4-layer CPU plumbing model: 3 Gated DeltaNet + 1 gated full-attention
    layer, hidden 256, FFN 704, 4 Q / 2 KV heads of 64, DeltaNet 2 QK / 4 V
    heads of 64, vocab 1024, partial RoPE over 16 dims, theta 1e7."""
    kw = dict(
        hidden_size=256, intermediate_size=704, num_hidden_layers=4,
        num_attention_heads=4, num_key_value_heads=2, head_dim=64,
        vocab_size=1024, max_position_embeddings=4096, rope_theta=1e7,
        rms_norm_eps=1e-6, full_attention_interval=4,
        linear_key_head_dim=64, linear_num_key_heads=2,
        linear_num_value_heads=4, linear_value_head_dim=64,
        linear_conv_kernel_dim=4, partial_rotary_factor=0.25,
        group_size=128, attn_quantized=True,
    )
    kw.update(overrides)
    return QwenConfig(**kw)


# (M, N, K, name) GEMM/GEMV shapes of the 27B model, used by the tuner and the
# micro-benchmarks (reference: src/model/qwen.py:117-137).
QWEN_GEMM_SHAPES = [
    (1, 2 * 6144 + 2 * 1024, 5120, "full_attn_qkv"),
    (512, 2 * 6144 + 2 * 1024, 5120, "full_attn_qkv_512"),
    (1, 2 * 2048 + 2 * 6144, 5120, "linear_attn_in_proj"),
    (512, 2 * 2048 + 2 * 6144, 5120, "linear_attn_in_proj_512"),
    (1, 5120, 6144, "attn_out_proj"),
    (512, 5120, 6144, "attn_out_proj_512"),
    (1, 2 * 17408, 5120, "ffn_gate_up"),
    (512, 2 * 17408, 5120, "ffn_gate_up_512"),
    (1, 5120, 17408, "ffn_down"),
    (512, 5120, 17408, "ffn_down_512"),
    (1, 248320, 5120, "lm_head"),
]


def load_config_from_json(model_dir: str) -> QwenConfig:
    path = Path(model_dir) / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"No config.json found in {model_dir}")
    hf = json.loads(path.read_text())
    text = hf.get("text_config", hf)
    rope = text.get("rope_parameters", {}) or {}
    names = {f.name for f in dataclasses.fields(QwenConfig)}
    kw = {k: text[k] for k in (
        "hidden_size", "intermediate_size", "num_hidden_layers",
        "num_attention_heads", "num_key_value_heads", "head_dim", "vocab_size",
        "max_position_embeddings", "rms_norm_eps", "full_attention_interval",
        "linear_key_head_dim", "linear_num_key_heads", "linear_num_value_heads",
        "linear_value_head_dim", "linear_conv_kernel_dim", "attn_output_gate",
        "rope_style",
    ) if k in text and k in names}
    if text.get("layer_types"):
        kw["layer_types"] = list(text["layer_types"])
    kw["rope_theta"] = rope.get("rope_theta", text.get("rope_theta", 1e7))
    kw["partial_rotary_factor"] = rope.get(
        "partial_rotary_factor", text.get("partial_rotary_factor", 0.25))
    if "mrope_section" in rope:
        kw["mrope_sections"] = list(rope["mrope_section"])
    kw["mrope_interleaved"] = rope.get("mrope_interleaved", True)
    cfg = QwenConfig(**kw)
    q = hf.get("quantization_config", text.get("quantization_config", {})) or {}
    if q:
        cfg.quant_method = q.get("quant_method", "gptq")
        cfg.bits = q.get("bits", q.get("num_bits", 4))
        cfg.group_size = q.get("group_size", 128)
        for grp in (q.get("config_groups") or {}).values():
            w = grp.get("weights", {}) or {}
            cfg.bits = w.get("num_bits", cfg.bits)
            cfg.group_size = w.get("group_size", cfg.group_size)
            cfg.quant_sym = w.get("symmetric", cfg.quant_sym)
        cfg.quant_sym = q.get("sym", True)
        dyn = q.get("dynamic", {}) or {}
        cfg.attn_quantized = "-:.*attn.*" not in dyn
    return cfg


def kv_cache_bytes(config: QwenConfig, max_seq_len: int, batch: int = 1,
                   tp_size: int = 1) -> int:
    """Bytes of fp16 K+V cache per rank.  Only full-attention layers keep one;
    with tp_size > num_key_value_heads each KV head lives on tp/kv ranks."""
    local_kv = max(1, config.num_key_value_heads // tp_size)
    per_layer = batch * max_seq_len * local_kv * config.head_dim * 2
    return 2 * config.num_full_attention_layers * per_layer


def deltanet_state_bytes(config: QwenConfig, batch: int = 1, tp_size: int = 1) -> int:
    vh = config.linear_num_value_heads // tp_size
    per = vh * config.linear_key_head_dim * config.linear_value_head_dim * 4
    conv = (config.linear_conv_dim // tp_size) * (config.linear_conv_kernel_dim - 1) * 2
    return config.num_linear_attention_layers * batch * (per + conv)


def memory_budget(config: QwenConfig, max_seq_len: int = 2048, num_gpus: int = 1,
                  batch: int = 1, int4_attention: Optional[bool] = None,
                  hbm_bytes: int = B200_HBM_BYTES) -> dict:
    """Per-GPU memory estimate (weights sharded by TP, embeddings replicated,
    lm_head vocab-sharded)."""
    int4_attn = config.attn_quantized if int4_attention is None else int4_attention
    h, inter = config.hidden_size, config.intermediate_size
    g = config.group_size
    n_full, n_lin = config.num_full_attention_layers, config.num_linear_attention_layers
    attn_params = n_full * h * (2 * config.full_attn_q_dim + 2 * config.full_attn_kv_dim
                                + config.full_attn_q_dim)
    lin_params = n_lin * h * (config.linear_conv_dim + 2 * config.linear_attn_value_dim)
    ffn_params = config.num_hidden_layers * 3 * h * inter

    def int4_bytes(p):
        return p // 2 + (p // g) * 2 + (p // g) // 2

    ffn_bytes = int4_bytes(ffn_params)
    attn_bytes = int4_bytes(attn_params + lin_params) if int4_attn else 2 * (attn_params + lin_params)
    embed_bytes = config.vocab_size * h * 2
    lm_head_bytes = config.vocab_size * h * 2
    sharded = ffn_bytes + attn_bytes + lm_head_bytes
    kv = kv_cache_bytes(config, max_seq_len, batch, num_gpus)
    dn = deltanet_state_bytes(config, batch, num_gpus)
    scratch = max_seq_len * h * 4 * 8
    per_gpu = sharded / num_gpus + embed_bytes + kv + dn + scratch
    total = sharded + embed_bytes + (kv + dn) * num_gpus + scratch
    return {
        "model_gb": (sharded + embed_bytes) / 1e9,
        "attn_gb": attn_bytes / 1e9,
        "ffn_int4_gb": ffn_bytes / 1e9,
        "kv_cache_gb_per_gpu": kv / 1e9,
        "deltanet_state_gb_per_gpu": dn / 1e9,
        "scratch_gb": scratch / 1e9,
        "total_gb": total / 1e9,
        "per_gpu_gb": per_gpu / 1e9,
        "fits_per_gpu": per_gpu < hbm_bytes,
        "min_gpus": max(1, int(-(-total // hbm_bytes))),
    }


AR_MODES = ("exact", "deferred_ref", "deferred_consistent")


@dataclass(frozen=True)
class EngineConfig:
    """How an engine runs.  `ar_mode`: 'exact' does two all-reduces per layer;
    'deferred_ref' reproduces the reference's deferred attention all-reduce
    (each rank adds only its own attention partial; reference:
    src/runtime/c_dispatch.c:1110-1121); 'deferred_consistent' sends the
    attention partial along with the FFN partial so the ranks' residual streams
    re-converge after every layer with one all-reduce per layer."""
    tp_size: int = 1
    tp_rank: int = 0
    max_seq_len: int = 2048
    max_batch: int = 1
    quant_format: str = "w4a16"
    use_int4_attention: bool = False
    ar_mode: str = "exact"
    use_graph: bool = True
    use_multimem: bool = True
    fused_gemv_ar: bool = True
    # the persistent projection-chain kernel (csrc/chain.cu) in the decode step: 0 off, 1 consecutive INT4
    # projections run as one launch, 2 only the projections that exchange across GPUs use it (one launch each),
    # -1 (default, or B200GRAD_CHAIN unset) = 2 on two to four GPUs, 0 otherwise
    use_chain: int = dataclasses.field(default_factory=lambda: int(os.environ.get("B200GRAD_CHAIN", "-1")))
    # many-row steps under tensor parallelism: 1 = residual stream sequence-parallel between the row-parallel
    # projections (reduce-scatter by token rows + norm + fp16 all-gather in one kernel), 0 = all-reduce + norm
    seq_parallel: int = dataclasses.field(default_factory=lambda: int(os.environ.get("B200GRAD_SEQ_PARALLEL", "1")))
    spec_ngram: int = 3
    spec_max_draft: int = 4
    max_step_rows: int = 0           # rows of a batched-decode / verify step (0: 8 per sequence slot)
    wait_budget_us: int = 2_000_000
    debug_guards: bool = False

    def __post_init__(self):
        if self.ar_mode not in AR_MODES:
            raise ValueError(f"ar_mode must be one of {AR_MODES}")
        if self.quant_format not in ("w4a16", "w8a8", "w4a8"):
            raise ValueError("quant_format must be w4a16, w8a8 or w4a8")

    def replace(self, **kw) -> "EngineConfig":
        return dataclasses.replace(self, **kw)

    @staticmethod
    def from_env(**kw) -> "EngineConfig":
        """Constructor kwargs overridden by B200GRAD_* environment variables."""
        env = os.environ
        if "B200GRAD_AR_MODE" in env:
            kw["ar_mode"] = env["B200GRAD_AR_MODE"]
        if "B200GRAD_GRAPH" in env:
            kw["use_graph"] = env["B200GRAD_GRAPH"] not in ("0", "false", "")
        if "B200GRAD_MULTIMEM" in env:
            kw["use_multimem"] = env["B200GRAD_MULTIMEM"] not in ("0", "false", "")
        if "B200GRAD_DEBUG_GUARDS" in env:
            kw["debug_guards"] = env["B200GRAD_DEBUG_GUARDS"] not in ("0", "false", "")
        return EngineConfig(**kw)
