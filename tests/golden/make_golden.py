"""Generates tests/golden/*.npz from the CPU oracle (run from the repository root:
python tests/golden/make_golden.py [tiny] [small]). The fixtures let the GPU tests check the
GPT-2-small-shaped configurations without re-running the minutes-long CPU oracle.

Contents per file:
  decode_<cfg>.npz : prompt ids, greedy tokens, top-2 margin of ln(max(p,1e-12)) per step,
                     and the log-prob of each emitted token
  score_<cfg>.npz  : ids of the first scoring sequences and their per-token log-probs
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from ferrum_cpu_b200 import synth  # noqa: E402
from tests import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
# name -> (prompt length, new tokens, scoring sequences kept, scoring sequence length)
PLAN = {"tiny": (16, 64, 4, 128), "small": (32, 256, 1, 1024), "medium": (64, 16, 1, 256)}


def make(name):
    n_prompt, n_new, n_seq, seq_len = PLAN[name]
    sm = synth.named(name, seed=0)
    V = sm.dims[5]
    om = O.OracleModel(sm, threads=os.cpu_count() or 1)
    prompt = synth.token_ids(0, n_prompt, V)
    t0 = time.time()
    toks, margin = om.generate_greedy(prompt, n_new)
    # log-prob of every emitted token under the distribution it was drawn from
    lps = []
    p = om.prime(prompt)
    for t in toks:
        lps.append(np.log(np.maximum(p[t], np.float32(1e-12))))
        p = om.feed(t)
    print(f"{name}: decode {time.time() - t0:.1f}s, min margin {margin.min():.3e}")
    np.savez_compressed(os.path.join(HERE, f"decode_{name}.npz"), prompt=prompt, tokens=toks, margin=margin,
                        token_logprob=np.array(lps, dtype=np.float32))
    ids = synth.token_ids(1, n_seq * seq_len, V).reshape(n_seq, seq_len)
    t0 = time.time()
    lp = np.zeros((n_seq, seq_len), dtype=np.float32)
    tot = np.zeros(n_seq)
    gr = np.zeros((n_seq, seq_len), dtype=np.uint8)
    for s in range(n_seq):
        tot[s], _, _, lp[s], gr[s] = om.token_logprobs(ids[s], 1)
    print(f"{name}: score {time.time() - t0:.1f}s, total logprob {tot}")
    np.savez_compressed(os.path.join(HERE, f"score_{name}.npz"), ids=ids, logprob=lp, total=tot, is_greedy=gr)


if __name__ == "__main__":
    for name in (sys.argv[1:] or list(PLAN)):
        make(name)
