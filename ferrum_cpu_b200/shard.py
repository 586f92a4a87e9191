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
    on_gpu = device is not None and torch.device(device).type == "cuda"
    # one staging buffer in pinned host memory, so that the copies to and from the device are single DMA transfers
    stage = torch.zeros((longest,) + local.shape[1:], dtype=torch.from_numpy(local[:0]).dtype, pin_memory=on_gpu)
    stage[:local.shape[0]] = torch.from_numpy(local)
    t = stage.to(device, non_blocking=True) if device is not None else stage
    parts = [torch.empty_like(t) for _ in range(world)] if rank == 0 else None
    dist.gather(t, parts, dst=0)
    if rank != 0:
        return None
    full = torch.empty((n_items,) + local.shape[1:], dtype=t.dtype, pin_memory=on_gpu)
    for r, part in enumerate(parts):
        a, b = shard_range(n_items, r, world)
        full[a:b].copy_(part[:b - a], non_blocking=True)
    if on_gpu:
        torch.cuda.synchronize(device)
    return full.numpy()


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
    # one record per sequence in one byte buffer, so that the path has ONE collective: [logprob, n_tokens, greedy]
    # as three f64, then the row of f32 log-probs
    T = ids2d.shape[1]
    head = np.array([[s.logprob, float(s.n_tokens), float(s.greedy)] for s in scores], dtype=np.float64).reshape(-1, 3)
    rec = np.zeros((b - a, 24 + 4 * T), dtype=np.uint8)
    rec[:, :24] = head.view(np.uint8).reshape(-1, 24)
    rec[:, 24:] = np.ascontiguousarray(lp, dtype=np.float32).view(np.uint8).reshape(-1, 4 * T)
    full = gather_rows(rec, n, rank, world, device)
    if rank != 0:
        return None
    head_all = np.ascontiguousarray(full[:, :24]).view(np.float64).reshape(-1, 3)
    lp_all = np.ascontiguousarray(full[:, 24:]).view(np.float32).reshape(-1, T)
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
