"""Draft-token trees and their attention masks.

A verification step feeds a whole tree of draft tokens through the model at
once; node i may attend to the committed context, to itself and to its
ancestors (reference: src/inference/tree_attention.py:186-208).  Besides the
dense mask the reference builds, `TreeAttentionMask.packed()` gives the
bit-packed per-node ancestor words the CUDA tree-verify attention kernel reads,
and `positions()` gives the RoPE position of each node (context length + depth;
the reference's engine hook fixes the position at 0:
src/inference/tp_engine.py:3186-3188).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np


class TreeNode:
    def __init__(self, token_id: int, parent: Optional["TreeNode"] = None):
        self.token_id = token_id
        self.parent = parent
        self.children: List["TreeNode"] = []
        self.depth = 0 if parent is None else parent.depth + 1
        self.index = -1

    def get_ancestors(self) -> List["TreeNode"]:
        out, n = [], self.parent
        while n is not None:
            out.append(n)
            n = n.parent
        return out

    def get_path_from_root(self) -> List["TreeNode"]:
        return list(reversed(self.get_ancestors())) + [self]

    def __repr__(self):
        return f"TreeNode(token={self.token_id}, depth={self.depth}, index={self.index})"


class TreeTopology:
    """Nodes are indexed in insertion order, which is breadth-first for the
    builders below, so a parent always precedes its children."""

    def __init__(self, root_token: int):
        self.root = TreeNode(root_token)
        self.nodes: List[TreeNode] = [self.root]
        self.root.index = 0

    def add_child(self, parent_node: TreeNode, token_id: int) -> TreeNode:
        n = TreeNode(token_id, parent_node)
        parent_node.children.append(n)
        n.index = len(self.nodes)
        self.nodes.append(n)
        return n

    def get_node_by_index(self, index: int) -> TreeNode:
        return self.nodes[index]

    def get_all_tokens(self) -> List[int]:
        return [n.token_id for n in self.nodes]

    def get_max_depth(self) -> int:
        return max(n.depth for n in self.nodes)

    def get_tree_size(self) -> int:
        return len(self.nodes)

    def get_nodes_at_depth(self, depth: int) -> List[TreeNode]:
        return [n for n in self.nodes if n.depth == depth]

    def parents(self) -> List[int]:
        """parent index per node, -1 for the root."""
        return [-1 if n.parent is None else n.parent.index for n in self.nodes]

    def depths(self) -> List[int]:
        return [n.depth for n in self.nodes]

    def to_dict(self) -> Dict:
        return {"size": len(self.nodes), "max_depth": self.get_max_depth(),
                "nodes": [{"index": n.index, "token_id": n.token_id, "depth": n.depth,
                           "parent": None if n.parent is None else n.parent.index,
                           "children": [c.index for c in n.children]} for n in self.nodes]}

    @classmethod
    def from_parents(cls, tokens: Sequence[int], parents: Sequence[int]) -> "TreeTopology":
        t = cls(tokens[0])
        for tok, p in zip(tokens[1:], parents[1:]):
            t.add_child(t.nodes[p], tok)
        return t


class TreeAttentionMask:
    """mask[i, j] over [tree, kv_len + tree]: columns < kv_len (context) are all
    visible; column kv_len + j is visible to node i iff j == i or j is an
    ancestor of i."""

    def __init__(self, tree_topology: TreeTopology, kv_len: int = 0):
        self.tree = tree_topology
        self.kv_len = kv_len
        self._tree_part = self._build_tree_part()

    def _build_tree_part(self) -> np.ndarray:
        T = self.tree.get_tree_size()
        m = np.zeros((T, T), dtype=bool)
        for n in self.tree.nodes:
            m[n.index, n.index] = True
            for a in n.get_ancestors():
                m[n.index, a.index] = True
        return m

    def get_mask(self) -> np.ndarray:
        T = self._tree_part.shape[0]
        return np.concatenate([np.ones((T, self.kv_len), dtype=bool), self._tree_part], axis=1)

    def get_causal_mask(self) -> np.ndarray:
        """What a chain of the same length would see (lower triangular)."""
        T = self._tree_part.shape[0]
        return np.concatenate([np.ones((T, self.kv_len), dtype=bool),
                               np.tril(np.ones((T, T), dtype=bool))], axis=1)

    def update_kv_len(self, kv_len: int):
        self.kv_len = kv_len

    def to_dense_int(self) -> np.ndarray:
        return self.get_mask().astype(np.int32)

    def packed(self) -> np.ndarray:
        """uint64 per node: bit j set iff node j is visible (tree part only;
        trees are limited to 64 nodes)."""
        T = self._tree_part.shape[0]
        if T > 64:
            raise ValueError("tree larger than 64 nodes")
        w = np.zeros(T, dtype=np.uint64)
        for i in range(T):
            for j in np.nonzero(self._tree_part[i])[0]:
                w[i] |= np.uint64(1) << np.uint64(j)
        return w

    def positions(self) -> np.ndarray:
        return self.kv_len + np.asarray(self.tree.depths(), dtype=np.int64)

    def visualize(self) -> str:
        rows = []
        for i, n in enumerate(self.tree.nodes):
            bits = "".join("#" if b else "." for b in self._tree_part[i])
            rows.append(f"{i:3d} d{n.depth} tok={n.token_id:<7d} [ctx x{self.kv_len}] {bits}")
        return "\n".join(rows)


def build_complete_binary_tree(root_token: int, depth: int, token_generator=None) -> TreeTopology:
    t = TreeTopology(root_token)
    nxt = [root_token + 1]

    def gen(parent, which):
        if token_generator is not None:
            return token_generator(parent, which)
        v = nxt[0]
        nxt[0] += 1
        return v
    frontier = [t.root]
    for _ in range(depth):
        new = []
        for p in frontier:
            for which in range(2):
                new.append(t.add_child(p, gen(p, which)))
        frontier = new
    return t


def build_chain_tree(token_ids: List[int]) -> TreeTopology:
    t = TreeTopology(token_ids[0])
    n = t.root
    for tok in token_ids[1:]:
        n = t.add_child(n, tok)
    return t


def build_star_tree(root_token: int, children_tokens: List[int]) -> TreeTopology:
    t = TreeTopology(root_token)
    for tok in children_tokens:
        t.add_child(t.root, tok)
    return t


def verify_tree_mask_correctness(mask: TreeAttentionMask, verbose: bool = False) -> bool:
    """Structural checks: context fully visible, diagonal set, visibility ==
    ancestor relation, nothing visible that comes later in index order."""
    m = mask.get_mask()
    kv, tree = mask.kv_len, mask.tree
    ok = bool(m[:, :kv].all())
    for n in tree.nodes:
        anc = {a.index for a in n.get_ancestors()} | {n.index}
        row = set(np.nonzero(m[n.index, kv:])[0].tolist())
        if row != anc:
            ok = False
            if verbose:
                print(f"node {n.index}: sees {sorted(row)}, expected {sorted(anc)}")
    return ok


def compare_tree_vs_sequential_attention(tree_mask: TreeAttentionMask, q: np.ndarray,
                                         k: np.ndarray, v: np.ndarray, atol: float = 1e-5) -> bool:
    """Masked attention over the tree must equal, for every node, plain causal
    attention over that node's root-to-node path.  q,k,v: [kv_len+tree, d] with
    the context rows first."""
    kv = tree_mask.kv_len
    m = tree_mask.get_mask()
    d = q.shape[1]
    for n in tree_mask.tree.nodes:
        i = kv + n.index
        sc = (k @ q[i]) / np.sqrt(d)
        sc = np.where(m[n.index], sc, -np.inf)
        p = np.exp(sc - sc.max())
        tree_out = (p / p.sum()) @ v
        rows = list(range(kv)) + [kv + a.index for a in n.get_path_from_root()]
        sc2 = (k[rows] @ q[i]) / np.sqrt(d)
        p2 = np.exp(sc2 - sc2.max())
        if not np.allclose(tree_out, (p2 / p2.sum()) @ v[rows], atol=atol):
            return False
    return True
