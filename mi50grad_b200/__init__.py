"""mi50grad_b200: a B200-native tensor-parallel inference engine for the
Qwen3.5 hybrid (Gated DeltaNet + gated full attention) decoder with INT4
weight-only quantisation."""
from .config import (EngineConfig, QwenConfig, kv_cache_bytes, load_config_from_json,
                     memory_budget, qwen35_27b, tiny_config, QWEN_GEMM_SHAPES)

__version__ = "0.1.0"
