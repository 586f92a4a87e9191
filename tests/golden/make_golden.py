"""Generates tests/golden/*.npz from the CPU oracle (run from the repository root:
python tests/golden/make_golden.py [tiny] [small] [medium] [streams-medium] [streams-small] [spread-small]).
The fixtures let the GPU tests check the GPT-2-small- and medium-shaped configurations without
re-running the minutes-long CPU oracle.

Contents per file:
  decode_<cfg>.npz         : prompt ids, greedy tokens, top-2 margin of ln(max(p,1e-12)) per step,
                             and the log-prob of each emitted token
  score_<cfg>.npz          : ids of the first scoring sequences and their per-token log-probs
  streams_<cfg>.npz        : for some of the concurrent decode streams of the batched-decode workload
                             (stream i's prompt is token_ids(200 + i, 64, V)): stream indices,
                             greedy tokens [n][new], top-2 margins [n][new]
  score_spread_small.npz   : eight of the 512 scoring sequences of the GPT-2-small workload
                             (first, last and six between): indices, ids, per-token log-probs
"""
import multiprocessing as mp
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
PLAN = {"tiny": (16, 64, 4, 128), "small": (32, 256, 1, 1024), "medium": (64, 128, 1, 1024)}
# concurrent-stream workload: model -> (stream indices, prompt length, new tokens)
STREAMS = {"medium": ([0, 9, 18, 27, 36, 45, 54, 63], 64, 128), "small": ([0, 1, 2, 3, 4, 5, 6, 7], 64, 128)}
STREAM_SEED = 200
SPREAD = [0, 73, 146, 219, 292, 365, 438, 511]


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
    print(f"{name}: decode {time.time() - t0:.1f}s, min margin {margin.min():.3e}", flush=True)
    np.savez_compressed(os.path.join(HERE, f"decode_{name}.npz"), prompt=prompt, tokens=toks, margin=margin,
                        token_logprob=np.array(lps, dtype=np.float32))
    ids = synth.token_ids(1, n_seq * seq_len, V).reshape(n_seq, seq_len)
    t0 = time.time()
    lp = np.zeros((n_seq, seq_len), dtype=np.float32)
    tot = np.zeros(n_seq)
    gr = np.zeros((n_seq, seq_len), dtype=np.uint8)
    for s in range(n_seq):
        tot[s], _, _, lp[s], gr[s] = om.token_logprobs(ids[s], 1)
    print(f"{name}: score {time.time() - t0:.1f}s, total logprob {tot}", flush=True)
    np.savez_compressed(os.path.join(HERE, f"score_{name}.npz"), ids=ids, logprob=lp, total=tot, is_greedy=gr)


def _one_stream(args):
    name, idx, n_prompt, n_new = args
    sm = synth.named(name, seed=0)
    om = O.OracleModel(sm, threads=1)          # one activation row: the reference runs it serially
    toks, margin = om.generate_greedy(synth.token_ids(STREAM_SEED + idx, n_prompt, sm.dims[5]), n_new)
    om.close()
    return idx, toks, margin[:n_new]


def make_streams(name):
    idxs, n_prompt, n_new = STREAMS[name]
    t0 = time.time()
    with mp.get_context("spawn").Pool(min(len(idxs), os.cpu_count() or 1)) as pool:
        res = pool.map(_one_stream, [(name, i, n_prompt, n_new) for i in idxs])
    toks = np.stack([r[1] for r in res])
    margin = np.stack([r[2] for r in res])
    print(f"streams-{name}: {time.time() - t0:.1f}s, min margin {margin.min():.3e}", flush=True)
    np.savez_compressed(os.path.join(HERE, f"streams_{name}.npz"), index=np.array(idxs, dtype=np.int32), prompt_len=n_prompt,
                        seed_base=STREAM_SEED, tokens=toks, margin=margin)


def make_spread_small():
    sm = synth.named("small", seed=0)
    V = sm.dims[5]
    ids_all = synth.token_ids(1, 512 * 1024, V).reshape(512, 1024)
    om = O.OracleModel(sm, threads=os.cpu_count() or 1)
    lp = np.zeros((len(SPREAD), 1024), dtype=np.float32)
    tot = np.zeros(len(SPREAD))
    t0 = time.time()
    for j, s in enumerate(SPREAD):
        tot[j], _, _, lp[j], _ = om.token_logprobs(ids_all[s], 1)
    print(f"spread-small: {time.time() - t0:.1f}s, totals {tot}", flush=True)
    np.savez_compressed(os.path.join(HERE, "score_spread_small.npz"), index=np.array(SPREAD, dtype=np.int32), ids=ids_all[SPREAD],
                        logprob=lp, total=tot)


if __name__ == "__main__":
    for name in (sys.argv[1:] or list(PLAN)):
        if name.startswith("streams-"):
            make_streams(name.split("-", 1)[1])
        elif name == "spread-small":
            make_spread_small()
        else:
            make(name)
