"""Text generation front-end (reference: src/inference/generate.py:23-397).

The reference's generator embeds tokens, applies the lm_head and samples on the
host, crossing PCIe twice per token per GPU.  Here greedy decoding stays on the
device (one graph replay per token); the host only uploads the chosen token and
downloads the next one, and for non-greedy sampling downloads nothing but the
sampled id (the sampler runs on the device when the engine offers it, else on
the gathered logits).
"""
from __future__ import annotations

import time
from typing import Callable, Iterator, List, Optional, Sequence

import numpy as np
import torch

from .sampler import SamplingParams, sample_token


class TextGenerator:
    def __init__(self, engine, embed_weight=None, lm_head_weight=None, tokenizer=None):
        """`engine`: InferenceEngine / TPInferenceEngine with weights loaded.
        embed_weight / lm_head_weight are accepted for signature compatibility and
        loaded into the engine when it has none."""
        self.engine = engine
        self.tokenizer = tokenizer
        core = getattr(engine, "engine", engine)
        if embed_weight is not None and core.embed is None:
            engine.load_embedding(torch.as_tensor(embed_weight))
        if lm_head_weight is not None and core.lm_head is None:
            engine.load_lm_head(torch.as_tensor(lm_head_weight))
        self.core = core

    # -- token-id level -----------------------------------------------------
    def _encode(self, prompt) -> List[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a tokenizer is needed for string prompts")
            return list(self.tokenizer.encode(prompt))
        return list(prompt)

    def _decode(self, ids: Sequence[int]) -> str:
        if self.tokenizer is None:
            return " ".join(str(i) for i in ids)
        return self.tokenizer.decode(list(ids))

    def prefill(self, token_ids: Sequence[int], seq: int = 0) -> int:
        """Consume the prompt; returns the greedy first token."""
        self.engine.reset(seq) if hasattr(self.engine, "reset") else self.core.states.reset(seq)
        return self.core.prefill_tokens(list(token_ids), seq)

    def stream_tokens(self, prompt_ids: Sequence[int], max_tokens: int,
                      params: Optional[SamplingParams] = None, seq: int = 0) -> Iterator[int]:
        params = params or SamplingParams(temperature=0.0, max_tokens=max_tokens)
        stop = set(params.stop_token_ids or [])
        greedy = params.temperature == 0 and params.repetition_penalty == 1.0
        past = list(prompt_ids)
        rng = np.random.default_rng(params.seed)
        # seed of the device sampler for this call: the caller's, or (unseeded, like the host path) a fresh one
        # from the host generator -- rank 0's under tensor parallelism, so that every rank draws the same tokens
        self._call_seed = params.seed if params.seed is not None else int(rng.integers(0, 2**31 - 1))
        if params.seed is None and getattr(self.engine, "tp_size", 1) > 1:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized():
                box = [self._call_seed]
                dist.broadcast_object_list(box, src=0)
                self._call_seed = int(box[0])
        tok = self.prefill(prompt_ids, seq)
        # on a GPU the sampler runs on the device (only the sampled id crosses PCIe); under tensor
        # parallelism every rank samples the all-gathered logits with the same seed, so all ranks draw
        # the same token without another exchange.  CPU engines sample on the host.
        on_device = (not greedy and params.temperature > 0 and torch.cuda.is_available()
                     and torch.device(getattr(self.core, "device", "cpu")).type == "cuda")
        draw = (lambda i: self._sample_device(params, past, i)) if on_device else \
            (lambda i: sample_token(self._full_logits(), params, past, rng))
        if not greedy:
            tok = draw(0)
        for i in range(max_tokens):
            yield tok
            past.append(tok)
            if tok in stop or i == max_tokens - 1:
                return
            nxt = self.core.step_host(tok, seq)
            tok = nxt if greedy else draw(i + 1)

    def _sample_device(self, params: SamplingParams, past: Sequence[int], step: int) -> int:
        from ..ops import kernels as K
        dev = self.core.device
        # the repetition penalty covers every distinct past token once, as the host sampler does
        uniq = sorted(set(int(t) for t in past))
        pt = torch.tensor([uniq], dtype=torch.int32, device=dev) if uniq else torch.zeros(1, 1, dtype=torch.int32, device=dev)
        npast = torch.tensor([len(uniq)], dtype=torch.int32, device=dev)
        seed = self._call_seed * 1000003 + step
        # the step left this rank's logits slice on the device; under tensor parallelism the ranks exchange
        # only their candidate lists (inside the sampling kernel) and draw the same token from the same seed:
        # no logits gather, no second lm_head pass, no collective call
        logits = self.core.logits(1)
        tp = getattr(self.engine, "tp_size", 1) > 1
        tok = K.sample_top_p(logits, params.temperature, params.top_k, params.top_p,
                             params.repetition_penalty, pt, npast, seed=seed,
                             vocab_offset=self.core.spec.vocab[0] if tp else 0,
                             comm=self.core._comm_ctx() if tp else None,
                             vocab_total=self.core.config.vocab_size if tp else 0)
        return int(tok[0].item())

    def _full_logits(self):
        lg = self.engine.compute_logits(None) if hasattr(self.engine, "tp_size") and self.engine.tp_size > 1 \
            else self.core.logits(1)[0]
        return lg.float().cpu().numpy() if isinstance(lg, torch.Tensor) else lg

    def generate_ids(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None) -> List[int]:
        params = params or SamplingParams()
        return list(self.stream_tokens(prompt_ids, params.max_tokens, params))

    # -- reference-compatible string level ------------------------------------
    def generate(self, prompt, params: Optional[SamplingParams] = None, stream: bool = False) -> str:
        params = params or SamplingParams()
        ids = self._encode(prompt)
        out = []
        for t in self.stream_tokens(ids, params.max_tokens, params):
            out.append(t)
            if stream:
                print(self._decode([t]), end="", flush=True)
        return self._decode(out)

    def generate_streaming(self, prompt, params: Optional[SamplingParams] = None,
                           callback: Optional[Callable[[str], None]] = None) -> Iterator[str]:
        params = params or SamplingParams()
        for t in self.stream_tokens(self._encode(prompt), params.max_tokens, params):
            piece = self._decode([t])
            if callback:
                callback(piece)
            yield piece

    def benchmark_ids(self, prompt_ids: Sequence[int], max_tokens: int = 100) -> dict:
        """Device-timed prefill and decode; every decode step uploads the token
        from pinned host memory and downloads the next one."""
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        torch.cuda.synchronize()
        ev[0].record()
        tok = self.prefill(prompt_ids)
        ev[1].record()
        n = 0
        for _ in range(max_tokens):
            tok = self.core.step_host(tok)
            n += 1
        ev[2].record()
        torch.cuda.synchronize()
        pre, dec = ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])
        return {"prompt_tokens": len(prompt_ids), "generated_tokens": n, "prefill_ms": pre, "decode_ms": dec,
                "ttft_ms": pre, "prefill_tok_s": len(prompt_ids) / (pre / 1e3),
                "decode_tok_s": n / (dec / 1e3), "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4}

    def benchmark(self, prompt, max_tokens: int = 100) -> dict:
        """(reference: src/inference/generate.py:193-248)"""
        return self.benchmark_ids(self._encode(prompt), max_tokens)

    def cleanup(self):
        self.engine.cleanup()


def _make_engine(model_dir: str, device_ids, max_seq_len: int):
    import torch.distributed as dist
    from ..engine.engine import InferenceEngine
    from ..engine.tp_engine import TPInferenceEngine
    from ..loaders import load_any
    loader = load_any(model_dir)
    cfg = loader.config
    tp = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    rank = dist.get_rank() if tp > 1 else 0
    if tp > 1:
        eng = TPInferenceEngine(cfg, device_ids, max_seq_len)
        for i in range(cfg.num_hidden_layers):
            eng.load_layer_weights(i, loader.load_layer(i, tp, rank), sharded=True)
        eng.load_lm_head(loader.load_lm_head(tp, rank), sharded=True)
    else:
        eng = InferenceEngine(cfg, (device_ids or [0])[0], max_seq_len)
        for i in range(cfg.num_hidden_layers):
            eng.load_layer_weights(i, loader.load_layer(i))
        eng.load_lm_head(loader.load_lm_head())
    eng.load_embedding(loader.load_embedding())
    eng.load_final_norm(loader.load_final_norm())
    return eng, loader


def load_and_generate(model_dir: str, prompt, device_ids=None, max_tokens: int = 256,
                      temperature: float = 0.7, max_seq_len: int = 4096, tokenizer=None) -> str:
    """Load a checkpoint directory (GPTQ / AWQ / compressed-tensors / fp16),
    generate, return the text (reference: src/inference/generate.py:257-320).
    Under torch.distributed every rank calls this and gets the same text."""
    eng, _ = _make_engine(model_dir, device_ids, max_seq_len)
    if tokenizer is None and isinstance(prompt, str):
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(model_dir, trust_remote_code=True)
    gen = TextGenerator(eng, tokenizer=tokenizer)
    try:
        return gen.generate(prompt, SamplingParams(temperature=temperature, max_tokens=max_tokens))
    finally:
        gen.cleanup()


def load_and_generate_eagle(model_dir: str, prompt, device_ids=None, max_tokens: int = 256,
                            temperature: float = 0.0, k_draft: int = 5, verbose: bool = False,
                            max_seq_len: int = 4096, tokenizer=None):
    """Load a checkpoint and generate with self-draft speculation: k_draft tokens are drafted from
    the model's own output head and verified in one pass (reference:
    src/inference/generate.py:323-397).  Decoding is greedy, so the text equals plain greedy
    generation; returns the text (token ids when there is no tokenizer)."""
    from .speculative import EagleSpeculativeGenerator
    if temperature != 0:
        raise ValueError("self-draft speculation here is greedy: temperature must be 0")
    eng, loader = _make_engine(model_dir, device_ids, max_seq_len)
    if tokenizer is None and isinstance(prompt, str):
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(model_dir, trust_remote_code=True)
    gen = EagleSpeculativeGenerator(eng, loader.load_embedding(), loader.load_lm_head(), tokenizer, k_draft=k_draft)
    try:
        out = gen.generate(prompt, SamplingParams(temperature=0.0, max_tokens=max_tokens), verbose=verbose)
        return out
    finally:
        gen.cleanup()
