"""Generates tests/golden/llama_1b.npz from the CPU oracle (run from the repository root:
python tests/golden/make_golden_llama.py). The fixture lets the GPU tests check the
Llama-3.2-1B-shaped model (synthetic weights, seed 0) without re-running the oracle, which
expands 1.04 G weights to f32 and takes minutes.

Contents: ids (the scored sequence), logprob (per-target ln softmax of llm_score.rs score_from,
window 2048), is_greedy, prompt / tokens / margin (greedy generation and the top-two logit gap
of the oracle at each step)."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from ferrum_cpu_b200 import synth  # noqa: E402
from tests import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    t0 = time.time()
    sm = synth.llama_named("llama-1b", seed=0)
    V = sm.dims["vocab"]
    om = O.OracleLlama(sm, threads=os.cpu_count() or 1)
    print(f"model built in {time.time() - t0:.0f}s")
    ids = synth.token_ids(1, 48, V)
    t0 = time.time()
    total, n, greedy, lp, gr = om.score_from(ids, 1, 2048)
    print(f"score {time.time() - t0:.0f}s: total {total:.6f} over {n}")
    prompt = synth.token_ids(0, 16, V)
    toks, margin = [], []
    om.clear()
    logits = None
    for t in prompt:
        logits = om.forward_one(t)
    t0 = time.time()
    for _ in range(8):
        top = np.sort(logits)[-2:]
        margin.append(float(top[1] - top[0]))
        tok = int(O.argmax_first(logits))
        toks.append(tok)
        logits = om.forward_one(tok)
    print(f"decode {time.time() - t0:.0f}s, min margin {min(margin):.3e}")
    np.savez_compressed(os.path.join(HERE, "llama_1b.npz"), ids=ids, logprob=lp.astype(np.float64), is_greedy=gr, total=total,
                        prompt=prompt, tokens=np.array(toks, dtype=np.int32), margin=np.array(margin, dtype=np.float32))


if __name__ == "__main__":
    main()
