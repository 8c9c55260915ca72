"""N-gram and self-draft ("EAGLE-style") speculative decoding.

Same public names as the reference (src/inference/speculative.py:24-890:
`NgramCache`, `speculative_decode`, `SpeculativeGenerator`, `EagleDraftHead`,
`eagle_speculative_decode`, `EagleSpeculativeGenerator`), different mechanics:

* the draft/verify loop talks to a *token backend* with one operation,
  `spec_step(root, drafts, parents)`: feed the pending token plus a draft chain or
  tree in ONE forward pass, accept the longest path the model itself would have
  produced greedily, and leave the sequence state exactly as if only the accepted
  tokens had been fed.  The reference verifies drafts with one forward pass per
  token and, on rejection, rewinds only a length counter, so its DeltaNet state
  keeps the rejected tokens (src/inference/tp_engine.py:1673-1687);
* greedy acceptance makes the output identical to plain greedy decoding; the
  tests check that equality token by token.
"""
from __future__ import annotations

import time
from collections import Counter, defaultdict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .sampler import SamplingParams


# ---------------------------------------------------------------------------
# n-gram cache
# ---------------------------------------------------------------------------
class NgramCache:
    """Index of every n-gram seen in the prompt and the generated text.

    Keys are (n-1)-token contexts, values count the tokens that followed them.
    `query` returns the continuations ordered by frequency, ties broken by most
    recent occurrence (reference: src/inference/speculative.py:24-120 keeps a
    nested-dict trie with unordered continuation lists).
    """

    def __init__(self, n: int = 3):
        if n < 2:
            raise ValueError("n-grams need n >= 2")
        self.n = n
        self.table: Dict[Tuple[int, ...], Counter] = defaultdict(Counter)
        self._last_seen: Dict[Tuple[int, ...], int] = {}
        self._clock = 0
        self._tail: List[int] = []          # last n-1 tokens indexed so far (for incremental updates)

    def __len__(self) -> int:
        return len(self.table)

    def _add(self, gram: Sequence[int]):
        ctx, nxt = tuple(gram[:-1]), int(gram[-1])
        self.table[ctx][nxt] += 1
        self._clock += 1
        self._last_seen[ctx + (nxt,)] = self._clock

    def build_from_sequence(self, tokens: Sequence[int]):
        tokens = [int(t) for t in tokens]
        for i in range(len(tokens) - self.n + 1):
            self._add(tokens[i:i + self.n])
        self._tail = tokens[-(self.n - 1):] if len(tokens) >= self.n - 1 else list(tokens)

    def update(self, new_tokens: Sequence[int]):
        """Index tokens appended to the sequence that was indexed before; n-grams
        that straddle the old end and the new tokens are included."""
        joined = self._tail + [int(t) for t in new_tokens]
        for i in range(len(joined) - self.n + 1):
            self._add(joined[i:i + self.n])
        self._tail = joined[-(self.n - 1):]

    def clear(self):
        self.table.clear()
        self._last_seen.clear()
        self._tail = []
        self._clock = 0

    def query(self, context: Sequence[int]) -> Optional[List[int]]:
        if len(context) < self.n - 1:
            return None
        ctx = tuple(int(t) for t in context[-(self.n - 1):])
        c = self.table.get(ctx)
        if not c:
            return None
        return sorted(c, key=lambda t: (-c[t], -self._last_seen[ctx + (t,)]))

    def draft_chain(self, context: Sequence[int], max_len: int) -> List[int]:
        """Most likely continuation, one token at a time, up to max_len."""
        ctx = [int(t) for t in context]
        out: List[int] = []
        for _ in range(max_len):
            c = self.query(ctx)
            if not c:
                break
            out.append(c[0])
            ctx.append(c[0])
        return out

    def generate_tree_drafts(self, context: Sequence[int], max_tree_size: int = 7, max_depth: int = 2,
                             branching_factor: int = 2) -> Dict:
        """Breadth-first draft tree.  Returns {'tokens': [...], 'parents': [...],
        'depths': [...]} with parent -1 = child of the last context token."""
        tokens: List[int] = []
        parents: List[int] = []
        depths: List[int] = []
        frontier: List[Tuple[int, List[int]]] = [(-1, [int(t) for t in context])]
        depth = 0
        while frontier and depth < max_depth and len(tokens) < max_tree_size:
            nxt_frontier = []
            for parent, ctx in frontier:
                for t in (self.query(ctx) or [])[:branching_factor]:
                    if len(tokens) >= max_tree_size:
                        break
                    tokens.append(t)
                    parents.append(parent)
                    depths.append(depth + 1)
                    nxt_frontier.append((len(tokens) - 1, ctx + [t]))
            frontier = nxt_frontier
            depth += 1
        return {"tokens": tokens, "parents": parents, "depths": depths}


# ---------------------------------------------------------------------------
# token backends
# ---------------------------------------------------------------------------
def accept_path(out_tokens: Sequence[int], root_out: int, drafts: Sequence[int], parents: Sequence[int]):
    """Greedy acceptance on the host.  `root_out` is the model's prediction after
    the pending token, out_tokens[i] its prediction after draft i.  Returns
    (indices of the accepted drafts in path order, next token)."""
    path: List[int] = []
    cur, pred = -1, int(root_out)
    while True:
        nxt = next((i for i, (t, p) in enumerate(zip(drafts, parents)) if p == cur and int(t) == pred), None)
        if nxt is None:
            return path, pred
        path.append(nxt)
        cur, pred = nxt, int(out_tokens[nxt])


class OracleBackend:
    """Token backend over the fp32 CPU model (models.oracle.OracleEngine)."""

    def __init__(self, oracle, seq: int = 0):
        self.o, self.seq = oracle, seq
        self.forward_passes = 0

    def reset(self):
        self.o.reset(self.seq)

    def _greedy(self, x: torch.Tensor) -> List[int]:
        logits = self.o.compute_logits(self.o.final_norm(x))
        return [int(t) for t in torch.argmax(logits, dim=-1)]

    def prefill(self, tokens: Sequence[int]) -> int:
        self.forward_passes += 1
        return self._greedy(self.o.forward(self.o.embed(list(tokens)), self.seq))[-1]

    def spec_step(self, root: int, drafts: Sequence[int], parents: Sequence[int]) -> Tuple[List[int], int]:
        toks = [int(root)] + [int(t) for t in drafts]
        if not drafts:
            self.forward_passes += 1
            return [], self._greedy(self.o.forward(self.o.embed(toks), self.seq))[-1]
        par = [-1] + [p + 1 for p in parents]
        self.forward_passes += 1
        outs = self._greedy(self.o.forward(self.o.embed(toks), self.seq, parents=par))
        path, nxt = accept_path(outs[1:], outs[0], drafts, parents)
        accepted = [int(drafts[i]) for i in path]
        # commit: the tree pass left the state untouched; feed the accepted chain
        self.o.forward(self.o.embed([int(root)] + accepted), self.seq)
        return accepted, nxt


class EngineBackend:
    """Token backend over InferenceEngine / TPInferenceEngine.  Uses the engine's
    one-pass verify-and-commit step when it has one (`spec_step_tokens`), else a
    dry-run chain pass followed by a committing pass of the accepted tokens."""

    def __init__(self, engine, seq: int = 0):
        self.e, self.seq = engine, seq
        self.forward_passes = 0

    def reset(self):
        self.e.reset(self.seq)

    def prefill(self, tokens: Sequence[int]) -> int:
        self.forward_passes += 1
        return int(self.e.prefill_tokens(list(tokens), self.seq))

    def spec_step(self, root: int, drafts: Sequence[int], parents: Sequence[int]) -> Tuple[List[int], int]:
        drafts = [int(t) for t in drafts]
        fused = getattr(self.e, "spec_step_tokens", None)
        if fused is not None:
            self.forward_passes += 1
            return fused(int(root), drafts, list(parents), self.seq)
        is_chain = all(p == i - 1 for i, p in enumerate(parents))
        if not drafts or not is_chain:
            self.forward_passes += 1
            out = self.e.step_tokens([int(root)], self.seq)
            return [], int(out[0].item())
        self.forward_passes += 2
        outs = self.e.step_tokens([int(root)] + drafts, self.seq, commit=False).tolist()
        path, nxt = accept_path(outs[1:], outs[0], drafts, parents)
        accepted = [drafts[i] for i in path]
        self.e.step_tokens([int(root)] + accepted, self.seq, logits=False)
        return accepted, nxt


def make_backend(engine, seq: int = 0):
    if hasattr(engine, "spec_step") and hasattr(engine, "prefill"):
        return engine
    if hasattr(engine, "greedy_generate") and hasattr(engine, "forward"):
        return OracleBackend(engine, seq)
    return EngineBackend(engine, seq)


# ---------------------------------------------------------------------------
# n-gram speculative decoding
# ---------------------------------------------------------------------------
@dataclass
class SpecStats:
    iterations: int = 0
    drafted: int = 0
    accepted: int = 0
    generated: int = 0
    forward_passes: int = 0
    seconds: float = 0.0
    per_iteration: List[int] = field(default_factory=list)

    def as_dict(self) -> dict:
        return {
            "iterations": self.iterations, "draft_tokens": self.drafted, "accepted_tokens": self.accepted,
            "generated_tokens": self.generated, "forward_passes": self.forward_passes,
            "acceptance_rate": self.accepted / self.drafted if self.drafted else 0.0,
            "tokens_per_iteration": self.generated / self.iterations if self.iterations else 0.0,
            "seconds": self.seconds,
            "tokens_per_second": self.generated / self.seconds if self.seconds > 0 else 0.0,
        }


def speculative_decode(generator, input_ids: Sequence[int], params: Optional[SamplingParams],
                       ngram_cache: Optional[NgramCache] = None, ngram_size: int = 3, max_draft_len: int = 5,
                       token_id_key: str = "token_id", verbose: bool = False) -> Tuple[List[int], dict]:
    """Draft with n-gram look-ups, verify a whole draft in one pass, keep the
    longest prefix the model agrees with (reference:
    src/inference/speculative.py:231-417).  `generator` is a token backend, an
    engine, or anything with a `.backend` attribute.  Decoding is greedy: with a
    temperature the drafts could not be accepted by token equality."""
    backend = getattr(generator, "backend", None) or make_backend(getattr(generator, "engine", generator))
    params = params or SamplingParams(temperature=0.0)
    if params.temperature != 0:
        raise ValueError("speculative decoding here is greedy (temperature 0)")
    cache = ngram_cache if ngram_cache is not None else NgramCache(ngram_size)
    stop = set(params.stop_token_ids or [])
    stats = SpecStats()
    t0 = time.perf_counter()
    fp0 = getattr(backend, "forward_passes", 0)
    context = [int(t) for t in input_ids]
    cache.build_from_sequence(context)
    backend.reset()
    pending = backend.prefill(context)
    out: List[int] = []
    while len(out) < params.max_tokens:
        # `pending` is decided but not fed yet
        room = params.max_tokens - len(out) - 1
        drafts = cache.draft_chain(context + [pending], min(max_draft_len, max(room, 0)))
        accepted, nxt = backend.spec_step(pending, drafts, list(range(-1, len(drafts) - 1)))
        new = [pending] + accepted
        stats.iterations += 1
        stats.drafted += len(drafts)
        stats.accepted += len(accepted)
        stats.per_iteration.append(len(new))
        if verbose:
            print(f"[spec] drafts={drafts} accepted={accepted} next={nxt}")
        hit_stop = False
        for t in new:
            out.append(t)
            if t in stop or len(out) >= params.max_tokens:
                hit_stop = True
                break
        cache.update(new)
        context.extend(new)
        pending = nxt
        if hit_stop:
            break
    stats.generated = len(out)
    stats.seconds = time.perf_counter() - t0
    stats.forward_passes = getattr(backend, "forward_passes", 0) - fp0
    return out, stats.as_dict()


class SpeculativeGenerator:
    """Generator front-end with n-gram speculation (reference:
    src/inference/speculative.py:420-524)."""

    def __init__(self, engine, embed_weight=None, lm_head_weight=None, tokenizer=None,
                 ngram_size: int = 3, max_draft_len: int = 5):
        core = getattr(engine, "engine", engine)
        if embed_weight is not None and getattr(core, "embed", True) is None:
            engine.load_embedding(torch.as_tensor(embed_weight))
        if lm_head_weight is not None and getattr(core, "lm_head", True) is None:
            engine.load_lm_head(torch.as_tensor(lm_head_weight))
        self.engine, self.tokenizer = engine, tokenizer
        self.backend = make_backend(engine)
        self.ngram_size, self.max_draft_len = ngram_size, max_draft_len
        self.last_stats: dict = {}

    def _ids(self, prompt) -> List[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a tokenizer is needed for string prompts")
            return list(self.tokenizer.encode(prompt))
        return [int(t) for t in prompt]

    def generate_ids(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None) -> List[int]:
        params = params or SamplingParams(temperature=0.0)
        ids, self.last_stats = speculative_decode(self, prompt_ids, params, NgramCache(self.ngram_size),
                                                  self.ngram_size, self.max_draft_len)
        return ids

    def generate(self, prompt, params: Optional[SamplingParams] = None, verbose: bool = False):
        ids = self.generate_ids(self._ids(prompt), params)
        if verbose:
            print(self.last_stats)
        return self.tokenizer.decode(ids) if self.tokenizer is not None else ids

    def benchmark(self, prompt, max_tokens: int = 100, verbose: bool = False) -> dict:
        self.generate_ids(self._ids(prompt), SamplingParams(temperature=0.0, max_tokens=max_tokens))
        if verbose:
            print(self.last_stats)
        return dict(self.last_stats)

    def cleanup(self):
        if hasattr(self.engine, "cleanup"):
            self.engine.cleanup()


# ---------------------------------------------------------------------------
# self-draft ("EAGLE-style") speculation
# ---------------------------------------------------------------------------
class EagleDraftHead:
    """Draft tokens from the model's own output head: token = argmax(lm_head(h)),
    then h <- normalised embedding of that token, repeated k times (reference:
    src/inference/speculative.py:526-627).  There is no trained draft network in
    either code base, so after the first token (which is the model's real
    prediction) the drafts are a heuristic; verification keeps the output exact."""

    def __init__(self, embed_weight, lm_head_weight, k_draft: int = 5, temperature: float = 0.0,
                 final_norm_weight=None, eps: float = 1e-6):
        self.embed = torch.as_tensor(np.asarray(embed_weight) if not torch.is_tensor(embed_weight) else embed_weight).float()
        self.lm_head = torch.as_tensor(np.asarray(lm_head_weight) if not torch.is_tensor(lm_head_weight) else lm_head_weight).float()
        self.k_draft, self.temperature, self.eps = k_draft, temperature, eps
        self.norm_w = None if final_norm_weight is None else torch.as_tensor(final_norm_weight).float()

    def _apply_lm_head(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.lm_head @ hidden

    def _sample_logits(self, logits: torch.Tensor, temperature: float = 0.0, rng=None) -> int:
        if temperature <= 0:
            return int(torch.argmax(logits))
        p = torch.softmax(logits / temperature, dim=-1).numpy().astype(np.float64)
        p /= p.sum()
        return int((rng or np.random.default_rng()).choice(len(p), p=p))

    def _norm(self, x: torch.Tensor) -> torch.Tensor:
        y = x * torch.rsqrt(x.pow(2).mean() + self.eps)
        return y * self.norm_w if self.norm_w is not None else y

    def generate_draft_tokens(self, hidden_state, k: Optional[int] = None, temperature: Optional[float] = None) -> List[int]:
        h = torch.as_tensor(np.asarray(hidden_state) if not torch.is_tensor(hidden_state) else hidden_state).float().flatten()
        temp = self.temperature if temperature is None else temperature
        out: List[int] = []
        for _ in range(self.k_draft if k is None else k):
            t = self._sample_logits(self._apply_lm_head(h), temp)
            out.append(t)
            h = self._norm(self.embed[t])
        return out


def eagle_speculative_decode(generator, input_ids: Sequence[int], params: Optional[SamplingParams],
                             draft_head: EagleDraftHead, k_draft: int = 5, verbose: bool = False,
                             hidden_fn=None) -> Tuple[List[int], dict]:
    """Draft k tokens with `draft_head` from the last hidden state, verify them in
    one pass (reference: src/inference/speculative.py:629-790).  `hidden_fn()`
    returns the final-normed hidden state of the last fed token; without it the
    draft head starts from the embedding of the pending token."""
    backend = getattr(generator, "backend", None) or make_backend(getattr(generator, "engine", generator))
    params = params or SamplingParams(temperature=0.0)
    if params.temperature != 0:
        raise ValueError("speculative decoding here is greedy (temperature 0)")
    stop = set(params.stop_token_ids or [])
    stats = SpecStats()
    t0 = time.perf_counter()
    fp0 = getattr(backend, "forward_passes", 0)
    backend.reset()
    pending = backend.prefill([int(t) for t in input_ids])
    out: List[int] = []
    while len(out) < params.max_tokens:
        room = params.max_tokens - len(out) - 1
        k = min(k_draft, max(room, 0))
        if k > 0:
            h = hidden_fn() if hidden_fn is not None else None
            if h is not None:
                # lm_head(h) reproduces `pending`; the drafts are what follows it
                drafts = draft_head.generate_draft_tokens(h, k + 1)[1:]
            else:
                drafts = draft_head.generate_draft_tokens(draft_head._norm(draft_head.embed[pending]), k)
        else:
            drafts = []
        accepted, nxt = backend.spec_step(pending, drafts, list(range(-1, len(drafts) - 1)))
        new = [pending] + accepted
        stats.iterations += 1
        stats.drafted += len(drafts)
        stats.accepted += len(accepted)
        if verbose:
            print(f"[eagle] drafts={drafts} accepted={accepted} next={nxt}")
        hit_stop = False
        for t in new:
            out.append(t)
            if t in stop or len(out) >= params.max_tokens:
                hit_stop = True
                break
        pending = nxt
        if hit_stop:
            break
    stats.generated = len(out)
    stats.seconds = time.perf_counter() - t0
    stats.forward_passes = getattr(backend, "forward_passes", 0) - fp0
    return out, stats.as_dict()


class EagleSpeculativeGenerator:
    """(reference: src/inference/speculative.py:792-890)"""

    def __init__(self, engine, embed_weight, lm_head_weight, tokenizer=None, k_draft: int = 5,
                 temperature: float = 0.0):
        self.engine, self.tokenizer = engine, tokenizer
        self.backend = make_backend(engine)
        self.k_draft = k_draft
        self.draft_head = EagleDraftHead(embed_weight, lm_head_weight, k_draft, temperature)
        self.last_stats: dict = {}

    def _ids(self, prompt) -> List[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a tokenizer is needed for string prompts")
            return list(self.tokenizer.encode(prompt))
        return [int(t) for t in prompt]

    def generate_ids(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None) -> List[int]:
        ids, self.last_stats = eagle_speculative_decode(self, prompt_ids, params or SamplingParams(temperature=0.0),
                                                        self.draft_head, self.k_draft)
        return ids

    def generate(self, prompt, params: Optional[SamplingParams] = None, verbose: bool = False):
        ids = self.generate_ids(self._ids(prompt), params)
        if verbose:
            print(self.last_stats)
        return self.tokenizer.decode(ids) if self.tokenizer is not None else ids

    def benchmark(self, prompt, max_tokens: int = 100, verbose: bool = False) -> dict:
        self.generate_ids(self._ids(prompt), SamplingParams(temperature=0.0, max_tokens=max_tokens))
        return dict(self.last_stats)

    def cleanup(self):
        if hasattr(self.engine, "cleanup"):
            self.engine.cleanup()
