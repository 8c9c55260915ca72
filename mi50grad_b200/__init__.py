"""mi50grad_b200: a B200-native tensor-parallel inference engine for the
Qwen3.5 hybrid (Gated DeltaNet + gated full attention) decoder with INT4
weight-only quantisation."""
from .config import (EngineConfig, QwenConfig, kv_cache_bytes, load_config_from_json,
                     memory_budget, qwen35_27b, tiny_config, QWEN_GEMM_SHAPES)

__version__ = "0.1.0"


def __getattr__(name):
    """Lazy access to the public API so that `import mi50grad_b200` stays light (no CUDA needed):
    InferenceEngine, TPInferenceEngine, TextGenerator, load_and_generate, SamplingParams,
    sample_token, OracleEngine, the weight loaders and detect_quant_format."""
    import importlib
    table = {
        "InferenceEngine": ".engine.engine", "TPInferenceEngine": ".engine.tp_engine",
        "TextGenerator": ".generate.generate", "load_and_generate": ".generate.generate",
        "SamplingParams": ".generate.sampler", "sample_token": ".generate.sampler",
        "SpeculativeGenerator": ".generate.speculative", "NgramCache": ".generate.speculative",
        "TreeSpeculativeDecoder": ".generate.tree_speculative", "OracleEngine": ".models.oracle",
        "QwenWeightLoader": ".loaders", "AWQWeightLoader": ".loaders", "CompressedTensorsLoader": ".loaders",
        "detect_quant_format": ".loaders", "load_awq_or_gptq": ".loaders",
        "TorchBaselineEngine": ".baseline.torch_engine",
    }
    if name in table:
        return getattr(importlib.import_module(table[name], __name__), name)
    raise AttributeError(name)
