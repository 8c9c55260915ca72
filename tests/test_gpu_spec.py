"""Speculative verification on the device against the fp32 oracle: tree verify, greedy
acceptance, exact commit of DeltaNet state / conv history / KV cache, many-row (tensor-core)
path, and batched decode of more sequences than the GEMV kernels take rows."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(max_batch, seed=0, max_seq=256):
    from mi50grad_b200.config import tiny_config
    from mi50grad_b200.engine.engine import InferenceEngine
    from mi50grad_b200.models.oracle import OracleEngine
    from mi50grad_b200.models.weights import random_model
    cfg = tiny_config()
    mw = random_model(cfg, seed)
    eng = InferenceEngine(cfg, max_seq_len=max_seq, max_batch=max_batch)
    eng.load_model(mw)
    return cfg, mw, eng, OracleEngine(mw, max_seq_len=max_seq, max_batch=max_batch)


def _prompt(cfg, n, seed):
    return torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _wrong(cfg, *avoid):
    t = 7
    while t in avoid:
        t += 1
    return t % cfg.vocab_size


def test_tree_verify_accepts_oracle_path_and_commits_exactly():
    cfg, mw, eng, orc = _mk(2)
    ids = _prompt(cfg, 12, 1)
    ref, _ = orc.greedy_generate(ids, 9)                  # ref[0] is the pending token after the prompt
    root = eng.prefill_tokens(ids)
    assert root == ref[0]
    g1, g2, g3 = ref[1], ref[2], ref[3]
    # node (draft index): 0 wrong, 1 g1 | below g1: 2 g2, 3 wrong | below g2: 4 wrong
    drafts = [_wrong(cfg, g1), g1, g2, _wrong(cfg, g2), _wrong(cfg, g3)]
    parents = [-1, -1, 1, 1, 2]
    (acc, nxt), = eng.spec_step([drafts], [parents], [0])
    assert acc == [g1, g2] and nxt == g3
    assert eng.states.length(0) == 12 + 3 and eng.states.token(0) == g3
    # the state must be what feeding root, g1, g2 one at a time leaves
    cfg2, _, eng2, _ = _mk(2)
    eng2.prefill_tokens(ids)
    eng2.decode_tokens(3, graph=False)
    S1, S2 = eng.states.dn.S[:, 0], eng2.states.dn.S[:, 0]
    assert (S1 - S2).abs().max() <= 2e-3 * max(1.0, S2.abs().max().item())
    assert torch.equal(eng.states.dn.conv[:, 0], eng2.states.dn.conv[:, 0])
    n = 15
    k1, k2 = eng.states.kv.k[:, 0, :n].float(), eng2.states.kv.k[:, 0, :n].float()
    assert (k1 - k2).abs().max() <= 2e-2 * max(1.0, k2.abs().max().item())
    # and decoding continues like the oracle
    cont = eng.decode_tokens(5, graph=False)[:, 0].tolist()
    assert [g3] + cont == ref[3:9]


def test_chain_speculation_through_generator_equals_greedy():
    from mi50grad_b200.generate.sampler import SamplingParams
    from mi50grad_b200.generate.speculative import SpeculativeGenerator
    from mi50grad_b200.generate.tree_speculative import TreeSpeculativeDecoder
    cfg, mw, eng, orc = _mk(1, seed=3)
    ids = ([11, 22, 33, 44, 55] * 4)[:18]
    ref, _ = orc.greedy_generate(ids, 20)
    gen = SpeculativeGenerator(eng, ngram_size=3, max_draft_len=4)
    out = gen.generate_ids(ids, SamplingParams(temperature=0.0, max_tokens=20))
    assert out == ref
    assert gen.last_stats["forward_passes"] == gen.last_stats["iterations"] + 1   # one pass per iteration + prefill
    dec = TreeSpeculativeDecoder(eng, max_tree_size=6, max_depth=3, branching_factor=2)
    assert dec.generate_ids(ids, 14) == ref[:14]


def test_many_row_verify_three_sequences_tensor_core_path():
    cfg, mw, eng, orc = _mk(4, seed=5)
    prompts = [_prompt(cfg, 17, 10), _prompt(cfg, 9, 11), _prompt(cfg, 20, 12)]
    refs = [orc.greedy_generate(p, 8, seq=i)[0] for i, p in enumerate(prompts)]
    for i, p in enumerate(prompts):
        assert eng.prefill_tokens(p, seq=i) == refs[i][0]
    drafts, parents, expect = [], [], []
    for i, r in enumerate(refs):
        n_ok = i                                           # sequence i accepts i drafts of a 3-chain
        d = [r[1 + k] if k < n_ok else _wrong(cfg, r[1 + k]) for k in range(3)]
        drafts.append(d)
        parents.append([-1, 0, 1])
        expect.append((d[:n_ok], r[1 + n_ok]))
    res = eng.spec_step(drafts, parents, [0, 1, 2])        # 12 rows: beyond the GEMV kernels' 8
    assert [(a, n) for a, n in res] == expect
    assert eng.states.lengths()[:3] == [17 + 1, 9 + 2, 20 + 3]
    out = eng.decode_tokens(3, seqs=[0, 1, 2], graph=False).cpu()
    for i, r in enumerate(refs):
        n_ok = i
        assert [r[1 + n_ok]] + out[:, i].tolist()[:2] == r[1 + n_ok:4 + n_ok][:3]


def test_batched_decode_more_sequences_than_gemv_rows():
    cfg, mw, eng, orc = _mk(10, seed=6, max_seq=64)
    prompts = [_prompt(cfg, 5 + i, 20 + i) for i in range(10)]
    refs = [orc.greedy_generate(p, 4, seq=i)[0] for i, p in enumerate(prompts)]
    for i, p in enumerate(prompts):
        assert eng.prefill_tokens(p, seq=i) == refs[i][0]
    out_e = eng.decode_tokens(3, seqs=list(range(10)), graph=False).cpu()
    for i in range(10):
        assert out_e[:, i].tolist() == refs[i][1:4], i
    assert eng.states.lengths() == [5 + i + 3 for i in range(10)]
    # the same step replayed from a captured graph
    out_g = eng.decode_tokens(2, seqs=list(range(10)), graph=True).cpu()
    assert out_g.shape == (2, 10)


def test_tp_engine_tree_hooks_match_oracle():
    from helpers import cosine
    from mi50grad_b200.config import tiny_config
    from mi50grad_b200.engine.tp_engine import TPInferenceEngine
    from mi50grad_b200.generate.tree_attention import TreeAttentionMask, TreeTopology
    from mi50grad_b200.models.oracle import OracleEngine
    from mi50grad_b200.models.weights import random_model
    cfg = tiny_config()
    mw = random_model(cfg, 4)
    eng = TPInferenceEngine(cfg, max_seq_len=128)
    eng.load_model(mw)
    orc = OracleEngine(mw, max_seq_len=128)
    ids = _prompt(cfg, 10, 31)
    eng.prefill_tokens(ids)
    orc.forward(orc.embed(ids))
    toks, parents = [5, 6, 7, 8, 9, 10], [-1, 0, 0, 1, 1, 2]
    topo = TreeTopology.from_parents(toks, parents)
    embs = orc.embed(toks)
    ref = orc.final_norm(orc.forward(embs, parents=parents))
    S_before = eng.engine.states.dn.S.clone()
    hs = eng.decode_step_tree([e.numpy() for e in embs], TreeAttentionMask(topo, kv_len=10))
    assert torch.equal(S_before, eng.engine.states.dn.S) and eng.engine.states.length(0) == 10
    for i in range(len(toks)):
        assert cosine(torch.from_numpy(hs[i]).float(), ref[i]) > 0.999, i
    hs2, n = eng.decode_step_speculative([e for e in embs[:3]], 10, [6, 7])
    ref2 = orc.final_norm(orc.forward(embs[:3], parents=[-1, 0, 1]))
    assert n == 2 and all(cosine(hs2[i].float().cpu(), ref2[i]) > 0.999 for i in range(3))
    eng.set_eagle_mode(True, k_draft=3)
    d = eng.generate_eagle_drafts(hs[0], 3)
    assert len(d) == 3 and d[0] == int(torch.argmax(orc.compute_logits(ref[0])))
