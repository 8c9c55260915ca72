import math

import torch

from mi50grad_b200.config import tiny_config
from mi50grad_b200.models import oracle as O
from mi50grad_b200.models.weights import random_model


def test_chunked_deltanet_equals_recurrent():
    g = torch.Generator().manual_seed(0)
    S, H, dk, dv = 150, 3, 32, 48
    q = O.l2norm(torch.randn(S, H, dk, generator=g)) / math.sqrt(dk)
    k = O.l2norm(torch.randn(S, H, dk, generator=g))
    v = torch.randn(S, H, dv, generator=g)
    gl = -torch.rand(S, H, generator=g) * 3
    gl[10] = -20.0
    beta = torch.rand(S, H, generator=g)
    s0 = torch.randn(H, dk, dv, generator=g) * 0.1
    s1, s2 = s0.clone(), s0.clone()
    y1 = O.deltanet_recurrent(q, k, v, gl, beta, s1)
    y2 = O.deltanet_chunked(q, k, v, gl, beta, s2, chunk=64)
    assert torch.allclose(y1, y2, atol=2e-5)
    assert torch.allclose(s1, s2, atol=2e-5)


def test_prefill_equals_token_by_token_and_chunked():
    cfg = tiny_config()
    mw = random_model(cfg, 0)
    ids = torch.randint(0, cfg.vocab_size, (21,), generator=torch.Generator().manual_seed(0)).tolist()
    a = O.OracleEngine(mw)
    xa = a.forward(a.embed(ids))
    b = O.OracleEngine(mw)
    xb = torch.stack([b.forward(b.embed([t]))[0] for t in ids])
    c = O.OracleEngine(mw, chunked_deltanet=True)
    xc = c.forward(c.embed(ids))
    scale = xa.abs().max()
    assert (xa - xb).abs().max() / scale < 1e-5
    assert (xa - xc).abs().max() / scale < 1e-5
    assert a.seqs[0].length == 21


def test_rope_styles_and_partial_rotation():
    cfg = tiny_config()
    cos, sin = O.rope_tables(cfg, torch.tensor([0, 5]))
    assert cos.shape == (2, cfg.rotary_dim // 2)
    x = torch.randn(2, 3, cfg.head_dim)
    for style in ("interleaved", "half"):
        y = O.apply_rope(x, cos, sin, style)
        assert torch.equal(y[..., cfg.rotary_dim:], x[..., cfg.rotary_dim:])
        assert torch.allclose(y[0], x[0], atol=1e-6)           # position 0 is the identity
        assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)


def test_tree_forward_matches_sequential_paths():
    cfg = tiny_config()
    mw = random_model(cfg, 1)
    e = O.OracleEngine(mw)
    ctx = [5, 9, 2, 77, 31]
    e.forward(e.embed(ctx))
    snap = e.snapshot()
    toks = [11, 12, 13, 14, 15]
    parents = [-1, 0, 0, 1, 2]           # two branches of depth 2 under node 0
    xt = e.forward(e.embed(toks), parents=parents)
    assert e.seqs[0].length == len(ctx)
    for leaf in (3, 4):
        path = []
        j = leaf
        while j >= 0:
            path.append(j)
            j = parents[j]
        path.reverse()
        e.restore(snap)
        xs = e.forward(e.embed([toks[j] for j in path]))
        for r, j in enumerate(path):
            assert (xs[r] - xt[j]).abs().max() / xs.abs().max() < 1e-5


def test_snapshot_restore_roundtrip():
    cfg = tiny_config()
    mw = random_model(cfg, 2)
    e = O.OracleEngine(mw)
    e.forward(e.embed([1, 2, 3]))
    snap = e.snapshot()
    a = e.forward(e.embed([4, 5]))
    e.restore(snap)
    b = e.forward(e.embed([4, 5]))
    assert torch.equal(a, b)


def test_oracle_score_tokens_matches_stepwise_logits():
    cfg = tiny_config()
    mw = random_model(cfg, 0)
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(3)).tolist()
    eng = O.OracleEngine(mw)
    lp = eng.score_tokens(ids)
    assert lp.shape == (11,) and bool((lp < 0).all())
    e2 = O.OracleEngine(mw)
    h = e2.prefill_step(e2.embed(ids[:5]))
    ref = torch.log_softmax(e2.compute_logits(h), -1)[ids[5]]
    assert abs(float(lp[4]) - float(ref)) < 1e-4
    assert 1.0 < eng.perplexity(ids) < 10 * cfg.vocab_size
