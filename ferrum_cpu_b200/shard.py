"""Batch partition over the GPUs of one box, above the C ABI.

The forward pass has no exchange step: scoring sequences and decode streams are independent,
weights are replicated, and item i goes to rank i * world // n_items (contiguous blocks). The
only collective is one gather of the results to rank 0. The reference scores requests one by
one on a single model thread (slm_server/src/model_thread.rs:29-38); this is the batch form of
that loop. Works on any torch.distributed backend (NCCL on GPUs, gloo in the CPU tests).
"""
import numpy as np


def shard_range(n_items, rank, world):
    """[start, stop) of the contiguous block of items that rank owns; blocks differ by at most one."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    return rank * n_items // world, (rank + 1) * n_items // world


def gather_rows(local, n_items, rank, world, device=None):
    """Gathers each rank's [rows_of_rank, ...] array to rank 0 in item order.

    Returns the full [n_items, ...] numpy array on rank 0 and None elsewhere. Blocks may have
    different lengths, so every rank pads to the longest block before the one gather.
    """
    local = np.ascontiguousarray(local)
    if world == 1:
        return local
    import torch
    import torch.distributed as dist
    longest = max(shard_range(n_items, r, world)[1] - shard_range(n_items, r, world)[0] for r in range(world))
    padded = np.zeros((longest,) + local.shape[1:], dtype=local.dtype)
    padded[:local.shape[0]] = local
    t = torch.from_numpy(padded)
    if device is not None:
        t = t.to(device)
    parts = [torch.empty_like(t) for _ in range(world)] if rank == 0 else None
    dist.gather(t, parts, dst=0)
    if rank != 0:
        return None
    out = []
    for r, part in enumerate(parts):
        a, b = shard_range(n_items, r, world)
        out.append(part[:b - a].cpu().numpy())
    return np.concatenate(out, axis=0)


def score_sharded(score_fn, ids2d, rank, world, device=None):
    """Scores this rank's block of sequences and gathers per-token log-probs and sequence sums.

    score_fn(ids_block) -> (list of objects with .logprob / .n_tokens / .greedy, lp [rows, T] f32),
    the shape of CudaSlm.score_sequences. Rank 0 gets (logprob [n] f64, n_tokens [n] i64,
    greedy [n] u8, lp [n, T] f32); the other ranks get None.
    """
    ids2d = np.ascontiguousarray(ids2d, dtype=np.int32)
    n = ids2d.shape[0]
    a, b = shard_range(n, rank, world)
    if b > a:
        scores, lp = score_fn(ids2d[a:b])
    else:
        scores, lp = [], np.zeros((0, ids2d.shape[1]), dtype=np.float32)
    # one record per sequence: [logprob, n_tokens, greedy] as f64, then the f32 rows
    head = np.array([[s.logprob, float(s.n_tokens), float(s.greedy)] for s in scores], dtype=np.float64).reshape(-1, 3)
    head_all = gather_rows(head, n, rank, world, device)
    lp_all = gather_rows(np.asarray(lp, dtype=np.float32), n, rank, world, device)
    if rank != 0:
        return None
    return head_all[:, 0], head_all[:, 1].astype(np.int64), head_all[:, 2].astype(np.uint8), lp_all


def decode_sharded(decode_fn, prompts2d, max_tokens, rank, world, device=None):
    """Runs this rank's block of decode streams and gathers the generated ids.

    decode_fn(prompts_block, max_tokens) -> list of int32 arrays (CudaSlm.decode_batch). Rank 0
    gets (tokens [n, max_tokens] i32 zero-padded, counts [n] i32); the other ranks get None.
    """
    prompts2d = np.ascontiguousarray(prompts2d, dtype=np.int32)
    n = prompts2d.shape[0]
    a, b = shard_range(n, rank, world)
    rows = decode_fn(prompts2d[a:b], max_tokens) if b > a else []
    toks = np.zeros((b - a, max(max_tokens, 1) + 1), dtype=np.int32)   # last column: the count
    for i, r in enumerate(rows):
        toks[i, :len(r)] = r
        toks[i, -1] = len(r)
    full = gather_rows(toks, n, rank, world, device)
    if rank != 0:
        return None
    return full[:, :-1], full[:, -1].copy()
