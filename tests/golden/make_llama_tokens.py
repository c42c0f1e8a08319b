#!/usr/bin/env python
"""Writes tests/golden/llama_config5_tokens.json: the greedy token stream of configuration 5
(22L / 2048 / 32q / 4kv / 5632 / 32000, seed 5, 512 LCG prompt ids, 128 greedy tokens) on ONE GPU,
after checking it against the float64 host forward of tests/llama_ref.py (teacher-forced, margin
gate as in tests/test_llama_full_size.py).  The file also records the float64 top-2 margin of
every step, so a reader can see which steps a different summation order could flip.

Needs a B200: run from the repository root as
    python tests/golden/make_llama_tokens.py [--out PATH]
"""
import argparse
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import __graft_entry__ as entry  # noqa: E402
from llama_ref import RefLlama, lcg_tokens  # noqa: E402

N_PROMPT, N_DECODE, TOL = 512, 128, 3e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "llama_config5_tokens.json"))
    args = ap.parse_args()
    ta, orc = entry.load_package(), entry.load_oracle()
    ctx = ta.Context(False, "index:0")
    ex = ta.Executor(ctx, 2, 1024)
    cfg = ta.LlamaConfig(t_max=1024, seed=5)
    model = ta.Llama(ex, cfg)
    prompt = lcg_tokens(N_PROMPT, cfg.vocab)
    nxt, _ = model.prefill(prompt)
    logits0 = model.logits()
    toks, _ = model.decode(nxt, N_DECODE)
    ref = RefLlama(orc, cfg, lean=True)
    want = ref.forward_positions(prompt + [nxt] + toks[:-1], N_DECODE + 1)
    got = [nxt] + toks
    margins, wrong = [], []
    for i in range(N_DECODE + 1):
        top = np.sort(want[i])[-2:]
        m = float((top[1] - top[0]) / np.abs(want[i]).max())
        margins.append(m)
        if m > 2 * TOL and got[i] != int(np.argmax(want[i])):
            wrong.append(i)
    e0 = float(np.abs(logits0.astype(np.float64) - want[0]).max() / np.abs(want[0]).max())
    if wrong or e0 > TOL:
        raise SystemExit(f"refusing to write a golden list: prefill rel err {e0:.3e}, wrong steps {wrong}")
    out = {"config": "llama 22L/2048/32q/4kv/5632/32000, weight seed 5, sigma 0.02, t_max 1024",
           "prompt_seed": 12345, "n_prompt": N_PROMPT, "tokens": got,
           "float64_top2_margin_rel": [round(m, 6) for m in margins],
           "margin_gate": 2 * TOL,
           "steps_under_margin_gate": [i for i, m in enumerate(margins) if m <= 2 * TOL],
           "prefill_logits_rel_err": e0}
    with open(args.out, "w") as f:
        json.dump(out, f, indent=1)
    print(f"wrote {args.out}: prefill rel err {e0:.2e}, {len(out['steps_under_margin_gate'])} low-margin steps")


if __name__ == "__main__":
    main()
