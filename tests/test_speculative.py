"""Host-side speculative decoding, prompt set, tuner database, step-graph IR (CPU)."""
import os

import torch

from mi50grad_b200.config import qwen35_27b, tiny_config
from mi50grad_b200.generate.prompts import (PromptCategory, PromptDataset, TrainTestSplitter, get_char_level_tokenizer,
                                            get_default_dataset, measure_ngram_acceptance)
from mi50grad_b200.generate.sampler import SamplingParams
from mi50grad_b200.generate.speculative import (EagleDraftHead, EagleSpeculativeGenerator, NgramCache, OracleBackend,
                                                SpeculativeGenerator, accept_path, speculative_decode)
from mi50grad_b200.generate.tree_speculative import TreeNgramPredictor, TreeSpeculativeDecoder, compare_tree_vs_greedy
from mi50grad_b200.graph.ir import build_step_graph
from mi50grad_b200.models.oracle import OracleEngine
from mi50grad_b200.models.weights import random_model
from mi50grad_b200.parallel.sharding import make_shard_spec
from mi50grad_b200.tune.tuner import TuneConfig, TuneDB, sweep


def test_ngram_cache_query_update_and_tree():
    c = NgramCache(3)
    c.build_from_sequence([1, 2, 3, 1, 2, 4, 1, 2, 4])
    assert c.query([9, 1, 2]) == [4, 3]            # 4 seen twice, 3 once
    assert c.query([7]) is None and c.query([5, 6]) is None
    c.update([5, 6])                               # n-grams across the old end: (2,4,5), (4,5,6)
    assert c.query([2, 4]) == [1, 5] or c.query([2, 4]) == [5, 1]
    assert c.query([4, 5]) == [6]
    assert c.draft_chain([1, 2], 3)[:1] == [4]
    t = c.generate_tree_drafts([1, 2], max_tree_size=5, max_depth=2, branching_factor=2)
    assert len(t["tokens"]) <= 5 and t["parents"][0] == -1 and set(t["tokens"][:2]) == {3, 4}
    assert all(p < i for i, p in enumerate(t["parents"]))
    c.clear()
    assert len(c) == 0


def test_accept_path_chain_and_tree():
    # chain: drafts 5,6,7; model says 5 after root, 6 after 5, 9 after 6
    path, nxt = accept_path([6, 9, 0], 5, [5, 6, 7], [-1, 0, 1])
    assert path == [0, 1] and nxt == 9
    # tree: two children of the root (4, 5); 5 is right; below 5 the child 8 is right
    path, nxt = accept_path([1, 8, 2, 3], 5, [4, 5, 7, 8], [-1, -1, 1, 1])
    assert path == [1, 3] and nxt == 3
    assert accept_path([], 3, [], []) == ([], 3)


def _oracle(seed=0):
    cfg = tiny_config()
    return cfg, random_model(cfg, seed)


def test_speculative_equals_greedy_oracle():
    cfg, mw = _oracle()
    prompt = ([3, 14, 15, 92, 65, 35] * 4)[:20]
    ref, _ = OracleEngine(mw).greedy_generate(prompt, 24)
    eng = OracleEngine(mw)
    gen = SpeculativeGenerator(eng, ngram_size=3, max_draft_len=4)
    out = gen.generate_ids(prompt, SamplingParams(temperature=0.0, max_tokens=24))
    assert out == ref
    st = gen.last_stats
    assert st["generated_tokens"] == 24 and st["iterations"] <= 24
    assert 0.0 <= st["acceptance_rate"] <= 1.0
    # the function form with a stop token
    out2, st2 = speculative_decode(OracleBackend(OracleEngine(mw)), prompt,
                                   SamplingParams(temperature=0.0, max_tokens=24, stop_token_ids=[ref[5]]))
    assert out2 == ref[:ref.index(ref[5]) + 1]


def test_speculative_accepts_on_repetitive_continuation():
    """A backend that just continues a periodic sequence: drafts must be accepted
    and the number of passes must drop."""
    class Periodic:
        def __init__(self, period):
            self.p, self.n, self.forward_passes = period, 0, 0
        def reset(self): self.n = 0
        def _tok(self, i): return self.p[i % len(self.p)]
        def prefill(self, toks):
            self.n = len(toks); self.forward_passes += 1
            return self._tok(self.n)
        def spec_step(self, root, drafts, parents):
            self.forward_passes += 1
            assert root == self._tok(self.n)
            outs = [self._tok(self.n + 1 + i) for i in range(len(drafts) + 1)]   # chain positions
            path, nxt = accept_path(outs[1:], outs[0], drafts, parents)
            self.n += 1 + len(path)
            return [drafts[i] for i in path], self._tok(self.n)
    period = [7, 8, 9, 10, 11]
    be = Periodic(period)
    out, st = speculative_decode(be, period * 3, SamplingParams(temperature=0.0, max_tokens=30), max_draft_len=4)
    assert out == [period[(15 + i) % 5] for i in range(30)]
    assert st["acceptance_rate"] == 1.0 and st["forward_passes"] <= 1 + 7


def test_tree_speculative_equals_greedy_oracle():
    cfg, mw = _oracle(1)
    prompt = ([5, 9, 2, 6] * 5)[:18]
    ref, _ = OracleEngine(mw).greedy_generate(prompt, 20)
    dec = TreeSpeculativeDecoder(OracleEngine(mw), max_tree_size=6, max_depth=3, branching_factor=2)
    assert dec.generate_ids(prompt, 20) == ref
    cmp = compare_tree_vs_greedy(dec, prompt, 12)
    assert cmp["match"] and cmp["tree_tokens"] == ref[:12]
    dec2 = TreeSpeculativeDecoder(OracleEngine(mw), max_tree_size=6, max_depth=3, use_optimizer=True)
    assert dec2.generate_ids(prompt, 10) == ref[:10]


def test_tree_predictor_shapes():
    c = NgramCache(2)
    c.build_from_sequence([1, 2, 1, 3, 1, 2, 2, 1])
    t = TreeNgramPredictor(c, 2).generate_tree([9, 1], None, max_tree_size=6, max_depth=2, branching_factor=2)
    assert t.root.token_id == 1 and {n.token_id for n in t.root.children} == {2, 3}
    assert t.get_tree_size() <= 7 and t.get_max_depth() <= 2
    shaped = TreeNgramPredictor(c, 2).generate_tree([9], 1, shape_parents=[-1, 0, 0, 1])
    assert shaped.parents()[:3] == [-1, 0, 0]


def test_eagle_generator_equals_greedy_oracle():
    cfg, mw = _oracle(2)
    prompt = list(range(10, 22))
    ref, _ = OracleEngine(mw).greedy_generate(prompt, 10)
    gen = EagleSpeculativeGenerator(OracleEngine(mw), mw.embed, mw.lm_head, k_draft=3)
    assert gen.generate_ids(prompt, SamplingParams(temperature=0.0, max_tokens=10)) == ref
    head = EagleDraftHead(mw.embed, mw.lm_head, k_draft=4)
    d = head.generate_draft_tokens(torch.randn(cfg.hidden_size))
    assert len(d) == 4 and all(0 <= t < cfg.vocab_size for t in d)


def test_prompt_dataset_roundtrip_and_split(tmp_path):
    d = PromptDataset()
    assert len(d) == 20 and all(len(d.get_prompts(c)) == 5 for c in PromptCategory)
    f = tmp_path / "p.json"
    d.save_to_file(str(f))
    d2 = PromptDataset.from_file(str(f))
    assert [p.text for p in d2.get_all_prompts()] == [p.text for p in d.get_all_prompts()]
    assert len(get_default_dataset()) == 20
    sp = TrainTestSplitter(0.6)
    tr, te = sp.split_tokens(list(range(100)))
    assert len(tr) == 60 and tr + te == list(range(100))
    tok = get_char_level_tokenizer()
    s = sp.split(d.get_prompts(PromptCategory.REPETITIVE)[0].text, tok)
    assert s.train_text + s.test_text == d.get_prompts(PromptCategory.REPETITIVE)[0].text
    assert tok.decode(tok.encode("héllo")) == "héllo"
    acc = measure_ngram_acceptance(d)
    assert acc["repetitive"] > acc["conversational"] > 0.0


def test_tune_db_and_sweep(tmp_path):
    db = TuneDB(str(tmp_path / "t.db"))
    cands = [TuneConfig.of(k_splits=s, L=l) for s in (1, 2, 4) for l in (2, 4)]
    cost = lambda c: 100.0 / c.as_dict()["k_splits"] + c.as_dict()["L"] if c.as_dict()["k_splits"] < 4 else float("inf")
    best = sweep("gemv_int4", 1, 5120, 17408, "int4", cands, cost, db, bytes_moved=44e6, device="test")
    assert best.config.as_dict() == {"k_splits": 2, "L": 2}
    got = db.best("gemv_int4", 1, 5120, 17408, "int4")
    assert got.config == best.config and abs(got.time_us - 52.0) < 1e-9 and got.gbytes_per_s > 0
    assert db.best("gemv_int4", 1, 1, 1, "int4") is None
    assert len(db.all("gemv_int4")) == 4
    db.close()


def test_step_graph_accounting():
    cfg = qwen35_27b()
    g = build_step_graph(cfg, make_shard_spec(cfg, 1, 0))
    s = g.summary()
    assert s["launches"] == 341 and s["collectives"] == 0
    assert 15.2e9 < s["weight_bytes"] < 15.7e9
    order = g.toposort()
    assert len(order) == len(g.ops) and order[0].name == "prepare_rows" and order[-1].name == "advance"
    g8 = build_step_graph(cfg, make_shard_spec(cfg, 8, 3))
    assert g8.summary()["collectives"] == 129
    gd = build_step_graph(cfg, make_shard_spec(cfg, 8, 3), ar_mode="deferred_ref")
    assert gd.summary()["collectives"] == 65
