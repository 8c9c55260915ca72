"""Tree-structured speculative decoding with n-gram drafts.

Public names follow the reference (src/inference/tree_speculative.py:31-686:
`TreeNgramPredictor`, `TreeSpeculativeDecoder`, `compare_tree_vs_greedy`).  What
differs: the whole draft tree is verified in one forward pass through a token
backend (`generate.speculative`), RoPE positions are length + depth, every node
continues from its parent's DeltaNet state, and the accepted path is committed
exactly.  The reference verifies a tree with position 0 for every node, lets the
DeltaNet layers ignore the tree and multiplies the lm_head on the host
(src/inference/tp_engine.py:3170-3236, tree_speculative.py:296-383).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Tuple

from .sampler import SamplingParams
from .speculative import NgramCache, SpecStats, make_backend
from .tree_attention import TreeNode, TreeTopology
from .tree_optimizer import SequoiaTreeOptimizer


class TreeNgramPredictor:
    """Grows a draft tree below the pending token from n-gram look-ups.  With
    `shape_parents` (e.g. the optimiser's topology) the tree follows that shape:
    the i-th child of a node takes the i-th most frequent continuation."""

    def __init__(self, ngram_cache: NgramCache, ngram_size: int = 3):
        self.cache, self.ngram_size = ngram_cache, ngram_size

    def _get_path_tokens(self, tree: TreeTopology, node: TreeNode) -> List[int]:
        return [n.token_id for n in node.get_path_from_root()]

    def generate_tree(self, context: Sequence[int], root_token: Optional[int] = None, max_tree_size: int = 7,
                      max_depth: int = 3, branching_factor: int = 2,
                      shape_parents: Optional[Sequence[int]] = None) -> TreeTopology:
        """Root = the pending token (`root_token`, default: last context token)."""
        context = [int(t) for t in context]
        if root_token is None:
            root_token, context = context[-1], context[:-1]
        tree = TreeTopology(int(root_token))
        if shape_parents is not None:
            return self._follow_shape(tree, context, shape_parents)
        frontier = [tree.root]
        while frontier and tree.get_tree_size() - 1 < max_tree_size:
            nxt = []
            for node in frontier:
                if node.depth >= max_depth:
                    continue
                cands = self.cache.query(context + self._get_path_tokens(tree, node)) or []
                for t in cands[:branching_factor]:
                    if tree.get_tree_size() - 1 >= max_tree_size:
                        break
                    nxt.append(tree.add_child(node, t))
            frontier = nxt
        return tree

    def _follow_shape(self, tree: TreeTopology, context: List[int], shape_parents: Sequence[int]) -> TreeTopology:
        # shape node 0 is the root; a shape node whose n-gram look-up has no candidate left is
        # dropped together with its subtree
        mapped: Dict[int, Optional[TreeNode]] = {0: tree.root}
        used: Dict[int, int] = {}
        for i in range(1, len(shape_parents)):
            parent = mapped.get(shape_parents[i])
            if parent is None:
                mapped[i] = None
                continue
            cands = self.cache.query(context + self._get_path_tokens(tree, parent)) or []
            k = used.get(parent.index, 0)
            if k >= len(cands):
                mapped[i] = None
                continue
            used[parent.index] = k + 1
            mapped[i] = tree.add_child(parent, cands[k])
        return tree

    def _build_optimized_tree_from_optimizer(self, context: Sequence[int], optimizer: SequoiaTreeOptimizer,
                                             root_token: Optional[int] = None) -> TreeTopology:
        return self.generate_tree(context, root_token, shape_parents=optimizer.find_optimal_tree().parents())


class TreeSpeculativeDecoder:
    def __init__(self, engine, embed_weight=None, lm_head_weight=None, tokenizer=None, ngram_size: int = 3,
                 max_tree_size: int = 7, max_depth: int = 3, branching_factor: int = 2,
                 use_optimizer: bool = False, optimizer: Optional[SequoiaTreeOptimizer] = None):
        """embed_weight / lm_head_weight are accepted for signature compatibility:
        embedding, lm_head and arg-max run inside the backend."""
        self.engine, self.tokenizer = engine, tokenizer
        self.backend = make_backend(engine)
        self.cache = NgramCache(ngram_size)
        self.predictor = TreeNgramPredictor(self.cache, ngram_size)
        self.max_tree_size, self.max_depth, self.branching_factor = max_tree_size, max_depth, branching_factor
        self.optimizer = optimizer or (SequoiaTreeOptimizer(max_depth=max_depth, max_branching=branching_factor,
                                                            size_budget=max_tree_size + 1) if use_optimizer else None)
        self._shape = self.optimizer.find_optimal_tree().parents() if self.optimizer else None
        self.context: List[int] = []
        self.pending: Optional[int] = None
        self.stats = SpecStats()

    # -- one iteration --------------------------------------------------------
    def start(self, prompt_ids: Sequence[int]):
        self.context = [int(t) for t in prompt_ids]
        self.cache.clear()
        self.cache.build_from_sequence(self.context)
        self.backend.reset()
        self.pending = self.backend.prefill(self.context)
        self.stats = SpecStats()

    def decode_step(self, max_new: Optional[int] = None) -> List[int]:
        """Draft a tree below the pending token, verify, commit the accepted
        path.  Returns the tokens that became final (pending + accepted)."""
        if self.pending is None:
            raise RuntimeError("call start(prompt_ids) first")
        budget = self.max_tree_size if max_new is None else max(0, min(self.max_tree_size, max_new - 1))
        depth = self.max_depth if max_new is None else max(0, min(self.max_depth, max_new - 1))
        if budget and depth:
            tree = self.predictor.generate_tree(self.context, self.pending, budget, depth, self.branching_factor,
                                                self._shape if max_new is None else None)
        else:
            tree = TreeTopology(self.pending)
        drafts = tree.get_all_tokens()[1:]
        parents = [p - 1 for p in tree.parents()[1:]]
        accepted, nxt = self.backend.spec_step(self.pending, drafts, parents)
        new = [self.pending] + accepted
        self.stats.iterations += 1
        self.stats.drafted += len(drafts)
        self.stats.accepted += len(accepted)
        self.stats.per_iteration.append(len(new))
        self.cache.update(new)
        self.context.extend(new)
        self.pending = nxt
        return new

    # -- loops ------------------------------------------------------------------
    def generate_ids(self, prompt_ids: Sequence[int], max_tokens: int = 100,
                     stop_token_ids: Optional[Sequence[int]] = None) -> List[int]:
        stop = set(stop_token_ids or [])
        t0 = time.perf_counter()
        fp0 = getattr(self.backend, "forward_passes", 0)
        self.start(prompt_ids)
        out: List[int] = []
        done = False
        while not done and len(out) < max_tokens:
            for t in self.decode_step(max_tokens - len(out)):
                out.append(t)
                if t in stop or len(out) >= max_tokens:
                    done = True
                    break
        self.stats.generated = len(out)
        self.stats.seconds = time.perf_counter() - t0
        self.stats.forward_passes = getattr(self.backend, "forward_passes", 0) - fp0
        return out

    def generate(self, prompt, params: Optional[SamplingParams] = None, verbose: bool = False):
        params = params or SamplingParams(temperature=0.0)
        if params.temperature != 0:
            raise ValueError("tree speculation here is greedy (temperature 0)")
        ids = list(self.tokenizer.encode(prompt)) if isinstance(prompt, str) else [int(t) for t in prompt]
        out = self.generate_ids(ids, params.max_tokens, params.stop_token_ids)
        if verbose:
            print(self.stats.as_dict())
        return self.tokenizer.decode(out) if (self.tokenizer is not None and isinstance(prompt, str)) else out

    def benchmark(self, prompt, max_tokens: int = 100, verbose: bool = False) -> dict:
        ids = list(self.tokenizer.encode(prompt)) if isinstance(prompt, str) else [int(t) for t in prompt]
        self.generate_ids(ids, max_tokens)
        d = self.stats.as_dict()
        d["tree_size_budget"] = self.max_tree_size
        if verbose:
            print(d)
        return d

    def cleanup(self):
        if hasattr(self.engine, "cleanup"):
            self.engine.cleanup()


def compare_tree_vs_greedy(tree_decoder: TreeSpeculativeDecoder, prompt_ids: Sequence[int],
                           max_tokens: int = 50) -> dict:
    """Run the tree decoder and plain greedy decoding (one token per pass through
    the same backend) and report whether the tokens agree and how many forward
    passes each needed (reference: src/inference/tree_speculative.py:634-686)."""
    be = tree_decoder.backend
    spec = tree_decoder.generate_ids(prompt_ids, max_tokens)
    spec_passes = tree_decoder.stats.forward_passes
    fp0 = getattr(be, "forward_passes", 0)
    be.reset()
    pending = be.prefill([int(t) for t in prompt_ids])
    greedy: List[int] = []
    while len(greedy) < max_tokens:
        greedy.append(pending)
        if len(greedy) == max_tokens:
            break
        _, pending = be.spec_step(pending, [], [])
    greedy_passes = getattr(be, "forward_passes", 0) - fp0
    return {"match": spec == greedy, "tree_tokens": spec, "greedy_tokens": greedy,
            "tree_forward_passes": spec_passes, "greedy_forward_passes": greedy_passes,
            "stats": tree_decoder.stats.as_dict()}
