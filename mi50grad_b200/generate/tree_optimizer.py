"""Sequoia-style dynamic programme for the draft-tree shape.

Maximises the expected number of accepted draft tokens for a node budget under
depth and branching limits, with the recurrence
    E(subtree rooted at depth d) = p(d) * (1 + sum of E(child subtrees))
(reference: src/inference/tree_optimizer.py:143-234).  The cost model is
re-based for NVLink: the reference prices a verification step at 64 all-reduces
of 46 us on PCIe (src/inference/tree_optimizer.py:76-83,111); the defaults here
are the same 64 all-reduces at a few microseconds, and `step_cost_ms` may be
replaced by a measured verify-step time.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from functools import lru_cache
from typing import Dict, Iterator, List, Optional, Sequence, Tuple


@dataclass
class TreeTopology:
    edges: List[Tuple[int, int]]
    num_nodes: int
    expected_tokens: float

    def parents(self) -> List[int]:
        p = [-1] * self.num_nodes
        for a, b in self.edges:
            p[b] = a
        return p

    def to_dict(self) -> Dict:
        return {"edges": [list(e) for e in self.edges], "num_nodes": self.num_nodes,
                "expected_tokens": self.expected_tokens}


class SequoiaTreeOptimizer:
    def __init__(self, base_acceptance_rate: float = 0.54, max_depth: int = 4,
                 max_branching: int = 2, size_budget: int = 16, acceptance_decay: float = 0.0,
                 allreduce_latency_us: float = 4.0, num_allreduces: int = 64,
                 acceptance_by_depth: Optional[Sequence[float]] = None):
        self.base_acceptance_rate = base_acceptance_rate
        self.max_depth = max_depth
        self.max_branching = max_branching
        self.size_budget = size_budget
        self.acceptance_decay = acceptance_decay
        self.allreduce_latency_us = allreduce_latency_us
        self.num_allreduces = num_allreduces
        self.verification_cost_ms = num_allreduces * allreduce_latency_us / 1000.0
        if acceptance_by_depth is not None:
            self._p = list(acceptance_by_depth)[:max_depth + 1]
            self._p += [self._p[-1]] * (max_depth + 1 - len(self._p))
        else:
            self._p = [base_acceptance_rate * (1.0 - acceptance_decay) ** d
                       if acceptance_decay > 0 else base_acceptance_rate
                       for d in range(max_depth + 1)]
        self._memo: Dict[Tuple[int, int], Tuple[float, Tuple[int, ...]]] = {}

    def get_acceptance_prob(self, depth: int) -> float:
        return self._p[depth] if 0 <= depth < len(self._p) else 0.0

    @staticmethod
    def _splits(total: int, parts: int) -> Iterator[Tuple[int, ...]]:
        """Non-increasing compositions (children are interchangeable)."""
        def rec(remaining, k, cap):
            if k == 1:
                if 1 <= remaining <= cap:
                    yield (remaining,)
                return
            for first in range(min(cap, remaining - (k - 1)), 0, -1):
                for rest in rec(remaining - first, k - 1, first):
                    yield (first,) + rest
        yield from rec(total, parts, total)

    def _solve(self, budget: int, depth: int) -> Tuple[float, Tuple[int, ...]]:
        if budget < 1 or depth > self.max_depth:
            return 0.0, ()
        key = (budget, depth)
        if key in self._memo:
            return self._memo[key]
        p = self.get_acceptance_prob(depth)
        best, best_children = p, ()
        child_budget = budget - 1
        if depth < self.max_depth:
            for used in range(1, child_budget + 1):
                for nc in range(1, min(self.max_branching, used) + 1):
                    for sizes in self._splits(used, nc):
                        e = p * (1.0 + sum(self._solve(s, depth + 1)[0] for s in sizes))
                        if e > best + 1e-12:
                            best, best_children = e, sizes
        self._memo[key] = (best, best_children)
        return self._memo[key]

    def _rebuild(self, budget: int, depth: int, edges: List[Tuple[int, int]], next_idx: List[int]) -> int:
        me = next_idx[0]
        next_idx[0] += 1
        for s in self._solve(budget, depth)[1]:
            child = self._rebuild(s, depth + 1, edges, next_idx)
            edges.append((me, child))
        return me

    def find_optimal_tree(self) -> TreeTopology:
        self._memo.clear()
        e, _ = self._solve(self.size_budget, 0)
        edges: List[Tuple[int, int]] = []
        n = [0]
        self._rebuild(self.size_budget, 0, edges, n)
        edges.sort(key=lambda ab: ab[1])
        return TreeTopology(edges, n[0], e)

    def chain_expectation(self, length: int) -> float:
        e, prod = 0.0, 1.0
        for d in range(length):
            prod *= self.get_acceptance_prob(min(d, self.max_depth))
            e += prod
        return e

    def compare_with_chain(self) -> Dict:
        tree = self.find_optimal_tree()
        L = min(self.size_budget, self.max_depth + 1)
        chain = self.chain_expectation(L)
        return {"tree_expected_tokens": tree.expected_tokens, "chain_expected_tokens": chain,
                "chain_length": L, "tree_nodes": tree.num_nodes,
                "improvement": tree.expected_tokens / chain if chain > 0 else float("inf"),
                "verification_cost_ms": self.verification_cost_ms,
                "tokens_per_ms_tree": (1.0 + tree.expected_tokens) / self.verification_cost_ms,
                "tokens_per_ms_chain": (1.0 + chain) / self.verification_cost_ms}

    def benchmark_runtime(self, num_runs: int = 10) -> Dict:
        ts = []
        for _ in range(num_runs):
            t0 = time.perf_counter()
            self.find_optimal_tree()
            ts.append((time.perf_counter() - t0) * 1e3)
        return {"mean_ms": sum(ts) / len(ts), "min_ms": min(ts), "max_ms": max(ts), "runs": num_runs}


def create_position_dependent_optimizer(acceptance_by_depth: Sequence[float], max_branching: int = 2,
                                        size_budget: int = 16, **kw) -> SequoiaTreeOptimizer:
    """Optimiser whose acceptance probability is given per depth (measured)."""
    return SequoiaTreeOptimizer(base_acceptance_rate=acceptance_by_depth[0],
                                max_depth=len(acceptance_by_depth) - 1,
                                max_branching=max_branching, size_budget=size_budget,
                                acceptance_by_depth=acceptance_by_depth, **kw)
