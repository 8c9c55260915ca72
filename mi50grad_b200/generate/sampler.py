"""Token sampling: repetition penalty -> temperature -> greedy if T == 0 ->
top-k -> softmax -> top-p -> multinomial, the order the reference applies them
(reference: src/inference/sampler.py:24-80).  The host version works on any
array-like of logits; the device version (ops.sample_top_p / ops.argmax) runs
the same pipeline on the GPU so that logits never cross PCIe during decode."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 50
    top_p: float = 0.9
    repetition_penalty: float = 1.0
    max_tokens: int = 256
    stop_token_ids: Optional[List[int]] = None
    seed: Optional[int] = None


def apply_repetition_penalty(logits: np.ndarray, past_tokens: Sequence[int], penalty: float):
    if past_tokens and penalty != 1.0:
        ids = np.fromiter({t for t in past_tokens if 0 <= t < logits.shape[0]}, dtype=np.int64)
        if ids.size:
            vals = logits[ids]
            logits[ids] = np.where(vals > 0, vals / penalty, vals * penalty)
    return logits


def filtered_probs(logits, params: SamplingParams, past_tokens=None) -> np.ndarray:
    """The distribution `sample_token` draws from (exposed for tests and for
    checking the GPU sampler)."""
    x = np.asarray(torch.as_tensor(logits).float().cpu().numpy() if isinstance(logits, torch.Tensor)
                   else logits, dtype=np.float32).copy()
    x = apply_repetition_penalty(x, past_tokens, params.repetition_penalty)
    if params.temperature > 0 and params.temperature != 1.0:
        x /= params.temperature
    if params.temperature == 0:
        p = np.zeros_like(x)
        p[int(np.argmax(x))] = 1.0
        return p
    if 0 < params.top_k < x.shape[0]:
        keep = np.argpartition(x, -params.top_k)[-params.top_k:]
        masked = np.full_like(x, -np.inf)
        masked[keep] = x[keep]
        x = masked
    x -= x.max()
    p = np.exp(x)
    p /= p.sum()
    if params.top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        csum = np.cumsum(p[order])
        cutoff = int(np.searchsorted(csum, params.top_p)) + 1
        kept = np.zeros_like(p)
        kept[order[:cutoff]] = p[order[:cutoff]]
        p = kept / kept.sum()
    return p


def sample_token(logits, params: SamplingParams, past_tokens: Optional[Sequence[int]] = None,
                 rng: Optional[np.random.Generator] = None) -> int:
    p = filtered_probs(logits, params, past_tokens)
    if params.temperature == 0:
        return int(np.argmax(p))
    if rng is None:
        rng = np.random.default_rng(params.seed) if params.seed is not None else np.random
    return int(rng.choice(p.shape[0], p=p))
