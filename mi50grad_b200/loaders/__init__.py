from .checkpoint import (AWQWeightLoader, CheckpointLoader, CompressedTensorsLoader,
                         QwenWeightLoader, awq_dequantize, detect_awq_format,
                         detect_compressed_tensors_format, detect_quant_format, load_any,
                         load_awq_or_gptq, load_compressed_tensors)
from .safetensors_io import CheckpointDir, SafetensorsFile, save_safetensors
