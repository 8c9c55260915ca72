import numpy as np
import torch

from mi50grad_b200.generate.sampler import SamplingParams, filtered_probs, sample_token
from mi50grad_b200.generate.tree_attention import (TreeAttentionMask, TreeTopology,
                                                   build_chain_tree, build_complete_binary_tree,
                                                   build_star_tree,
                                                   compare_tree_vs_sequential_attention,
                                                   verify_tree_mask_correctness)
from mi50grad_b200.generate.tree_optimizer import (SequoiaTreeOptimizer,
                                                   create_position_dependent_optimizer)


def test_greedy_and_repetition_penalty():
    logits = np.array([1.0, 3.0, 2.0, -1.0], dtype=np.float32)
    assert sample_token(logits, SamplingParams(temperature=0)) == 1
    p = SamplingParams(temperature=0, repetition_penalty=4.0)
    assert sample_token(logits, p, past_tokens=[1]) == 2
    neg = np.array([-1.0, -3.0], dtype=np.float32)
    assert sample_token(neg, p, past_tokens=[0]) == 1          # negative logits are multiplied


def test_top_k_top_p_support():
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    p = filtered_probs(logits, SamplingParams(top_k=0, top_p=0.75))
    assert np.count_nonzero(p) == 2 and abs(p.sum() - 1) < 1e-6
    p = filtered_probs(logits, SamplingParams(top_k=3, top_p=1.0))
    assert np.count_nonzero(p) == 3
    p = filtered_probs(torch.tensor(logits), SamplingParams(temperature=0.5, top_k=0, top_p=1.0))
    assert np.allclose(p, np.array([0.25, 0.09, 0.0225, 0.0025]) / 0.365, atol=1e-5)
    rng = np.random.default_rng(0)
    draws = [sample_token(logits, SamplingParams(top_k=2, top_p=1.0), rng=rng) for _ in range(200)]
    assert set(draws) <= {0, 1} and 80 < draws.count(0) < 170


def test_tree_masks():
    t = build_complete_binary_tree(1, 2)
    m = TreeAttentionMask(t, kv_len=3)
    assert m.get_mask().shape == (7, 10) and verify_tree_mask_correctness(m)
    assert list(m.packed()) == [1, 3, 5, 11, 19, 37, 69]
    assert list(m.positions()) == [3, 4, 4, 5, 5, 5, 5]
    chain = TreeAttentionMask(build_chain_tree([4, 5, 6]), 2)
    assert np.array_equal(chain.get_mask(), chain.get_causal_mask())
    star = build_star_tree(1, [2, 3, 4])
    assert star.parents() == [-1, 0, 0, 0] and star.get_max_depth() == 1
    assert TreeTopology.from_parents([1, 2, 3], [-1, 0, 1]).depths() == [0, 1, 2]
    rng = np.random.default_rng(0)
    n = 3 + 7
    q, k, v = (rng.standard_normal((n, 8)) for _ in range(3))
    assert compare_tree_vs_sequential_attention(m, q, k, v)
    m.update_kv_len(5)
    assert m.get_mask().shape == (7, 12)


def test_sequoia_dp():
    o = SequoiaTreeOptimizer(base_acceptance_rate=0.5, max_depth=3, max_branching=2, size_budget=7)
    t = o.find_optimal_tree()
    assert t.num_nodes <= 7 and len(t.edges) == t.num_nodes - 1
    par = t.parents()
    assert par[0] == -1 and all(0 <= par[i] < i for i in range(1, t.num_nodes))
    # expectation equals the sum over nodes of p^(depth+1) for uniform p
    depth = [0] * t.num_nodes
    for i in range(1, t.num_nodes):
        depth[i] = depth[par[i]] + 1
    assert abs(t.expected_tokens - sum(0.5 ** (d + 1) for d in depth)) < 1e-9
    assert max(depth) <= 3
    # a chain is optimal when branching is 1
    c = SequoiaTreeOptimizer(0.5, max_depth=3, max_branching=1, size_budget=4).find_optimal_tree()
    assert c.parents() == [-1, 0, 1, 2]
    cmp = o.compare_with_chain()
    assert cmp["tree_expected_tokens"] >= cmp["chain_expected_tokens"] - 1e-12
    pd = create_position_dependent_optimizer([0.9, 0.1, 0.1], max_branching=3, size_budget=4)
    assert pd.find_optimal_tree().expected_tokens > 0.9
    assert o.benchmark_runtime(2)["runs"] == 2
