"""The PyTorch/cuBLAS/NCCL baseline engine computes the same model (checked on CPU in fp32
against the oracle)."""
import torch

from mi50grad_b200.baseline.torch_engine import TorchBaselineEngine
from mi50grad_b200.config import tiny_config
from mi50grad_b200.models.oracle import OracleEngine
from mi50grad_b200.models.weights import random_model


def test_baseline_engine_matches_oracle_greedy():
    cfg = tiny_config()
    mw = random_model(cfg, 0)
    ids = torch.randint(0, cfg.vocab_size, (21,), generator=torch.Generator().manual_seed(2)).tolist()
    ref, _ = OracleEngine(mw).greedy_generate(ids, 7)
    eng = TorchBaselineEngine(cfg, device="cpu", max_seq_len=64, dtype=torch.float32)
    eng.load_model(mw)
    first = eng.prefill(ids)                      # 21 tokens: the chunked DeltaNet form
    rest = eng.decode(6, graph=False, collect=True)
    assert [first] + rest == ref
    short = ids[:9]                               # < 16 tokens: the recurrent form
    ref2, _ = OracleEngine(mw).greedy_generate(short, 4)
    assert [eng.prefill(short)] + eng.decode(3, graph=False, collect=True) == ref2
