"""The multi-GPU partition (one process per GPU, items split by index, one gather) run as two
gloo ranks on CPU: the scorer of each rank is the oracle, so the gathered result must equal the
unsharded one bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ferrum_cpu_b200 import shard, synth  # noqa: E402


def test_shard_ranges_cover_every_item_once():
    for n in (0, 1, 5, 64, 512, 1023):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                a, b = shard.shard_range(n, r, world)
                assert 0 <= a <= b <= n
                seen += list(range(a, b))
            assert seen == list(range(n))
            sizes = [shard.shard_range(n, r, world)[1] - shard.shard_range(n, r, world)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.shard_range(4, 2, 2)


class _S:
    def __init__(self, logprob, n_tokens, greedy):
        self.logprob, self.n_tokens, self.greedy = logprob, n_tokens, greedy


def _oracle_scorer():
    from tests import oracle
    sm = synth.SynthModel(2, 32, 2, 64, 16, 96, seed=4, perturb=True)
    om = oracle.OracleModel(sm)

    def score(block):
        scores, rows = [], []
        for ids in block:
            lp_sum, n, greedy, lp, _ = om.token_logprobs(ids, 1)
            scores.append(_S(lp_sum, n, greedy))
            rows.append(lp)
        return scores, np.stack(rows)

    def decode(block, max_tokens):
        return [np.asarray(om.generate_greedy(p, max_tokens)[0], dtype=np.int32) for p in block]

    return score, decode


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_seq, path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        score, decode = _oracle_scorer()
        ids = synth.token_ids(1, n_seq * 16, 96).reshape(n_seq, 16)
        got = shard.score_sharded(score, ids, rank, world)
        prompts = synth.token_ids(2, n_seq * 4, 96).reshape(n_seq, 4)
        dec = shard.decode_sharded(decode, prompts, 6, rank, world)
        if rank == 0:
            np.savez(path, logprob=got[0], n_tokens=got[1], greedy=got[2], lp=got[3], toks=dec[0], counts=dec[1])
        else:
            assert got is None and dec is None
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_seq", [4, 5])
def test_two_gloo_ranks_match_the_unsharded_scorer(tmp_path, n_seq):
    path = str(tmp_path / "out.npz")
    mp.spawn(_worker, args=(2, _free_port(), n_seq, path), nprocs=2, join=True)
    got = np.load(path)
    score, decode = _oracle_scorer()
    ids = synth.token_ids(1, n_seq * 16, 96).reshape(n_seq, 16)
    want = shard.score_sharded(score, ids, 0, 1)
    assert np.array_equal(got["logprob"], want[0]) and np.array_equal(got["n_tokens"], want[1])
    assert np.array_equal(got["greedy"], want[2]) and np.array_equal(got["lp"], want[3])
    prompts = synth.token_ids(2, n_seq * 4, 96).reshape(n_seq, 4)
    toks, counts = shard.decode_sharded(decode, prompts, 6, 0, 1)
    assert np.array_equal(got["toks"], toks) and np.array_equal(got["counts"], counts)
    assert (counts == 6).all()
