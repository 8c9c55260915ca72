"""Perplexity of a text or token file under a checkpoint (teacher forcing through the many-row
path).  The reference gates model quality on WikiText-2 perplexity in [5, 15] with no NaN
(reference: tests/eval_perplexity.py:1-16); datasets are not bundled here, so the text comes from a
file (or the packaged prompt set when none is given).

    python -m mi50grad_b200.bench.eval_perplexity /path/to/checkpoint --text file.txt --max-tokens 2048
"""
from __future__ import annotations

import argparse
import json
import math


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("model_dir")
    ap.add_argument("--text", default=None, help="UTF-8 text file (default: the packaged prompts)")
    ap.add_argument("--ids", default=None, help="JSON file with a list of token ids (no tokenizer needed)")
    ap.add_argument("--max-tokens", type=int, default=2048)
    ap.add_argument("--window", type=int, default=1024, help="tokens scored per sequence reset")
    a = ap.parse_args()
    from ..generate.generate import _make_engine
    eng, _ = _make_engine(a.model_dir, None, a.window + 8)
    if a.ids:
        ids = json.load(open(a.ids))
    else:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.model_dir, trust_remote_code=True)
        if a.text:
            text = open(a.text, encoding="utf-8").read()
        else:
            from ..generate.prompts import get_default_dataset
            text = "\n\n".join(p.text for p in get_default_dataset().get_all_prompts())
        ids = tok.encode(text)
    ids = [int(t) for t in ids][:a.max_tokens]
    import torch
    lps = []
    for i in range(0, len(ids) - 1, a.window):
        w = ids[i:i + a.window + 1]
        if len(w) > 1:
            lps.append(eng.score_tokens(w))
    lp = torch.cat(lps)
    ppl = math.exp(-float(lp.mean()))
    print(json.dumps({"tokens": int(lp.numel()), "perplexity": ppl, "nan": bool(torch.isnan(lp).any())}))


if __name__ == "__main__":
    main()
