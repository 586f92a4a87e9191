#!/usr/bin/env python
"""Benchmark of the Q8_0 GPT-2 forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode|score|both]
                    [--impl ours|reference]

Workloads (synthetic, seeded; shapes of the reference's configurations):
  decode : GPT-2-small-shaped Q8_0 model, batch 1, 32-token prompt, 256 greedy tokens with a
           KV cache. One step = one such generation. metric: decode tokens/s. At N GPUs every
           rank decodes its own stream (replicas only; the path does not shard).
  score  : the same model, 512 sequences x 1024 ids scored per step (per-token log-probs),
           sharded by sequence over the ranks with one gather of the results.

`value` is device time of the hot path with inputs resident (CUDA events on the launching
stream, max over ranks); `e2e` is the same metric through the C ABI with pinned host buffers,
host<->device copies and the prime inside the timed region. `--impl reference` times the CPU
restatement of the reference path (oracle/) on the host cores, on bounded samples.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

PROMPT, NEW_TOKENS = 32, 256
N_SEQ, SEQ_LEN = 512, 1024
METRIC = "Q8_0 GPT-2-small decode tokens/s (batch 1, KV cache, greedy)"
# dram__bytes_read.sum + dram__bytes_write.sum of decode_mega_kernel per token (ncu, see profiles/)
DECODE_DRAM_BYTES_PER_TOKEN = 134.8e6 + 4.98e6


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p.get("bf16_tflops_sustained", p["bf16_tflops"]), "measured"
    return 6650.0, 1400.0, "fallback"


def decode_bytes_per_token(dims, p_first, n_new):
    """Algorithmic HBM bytes of one KV-cached token, averaged over positions p_first..p_first+n_new-1:
    Q8_0 matrices once (34/32 B per weight), f32 biases/LayerNorm vectors, one position and one
    token row, f32 K/V rows read for positions 0..p and written for p."""
    L, d, H, F, T, V = dims
    q8 = (L * (4 * d * d + 2 * d * F) + d * V) * 34 // 32
    small = (L * (9 * d + F) + 2 * d) * 4 + d * 4 + d * 34 // 32
    kv = sum(L * 2 * (p + 1) * d * 4 + L * 2 * d * 4 for p in range(p_first, p_first + n_new)) / n_new
    return q8 + small + kv


def score_flops_per_position(dims):
    L, d, H, F, T, V = dims
    return 2 * (L * (4 * d * d + 2 * d * F) + d * V) + L * 4 * d * (T + 1) / 2


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        rows = [r for r in self.rows if len(r) == 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        busy = sorted(float(r[0]) for r in rows)
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": float(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def cpu_baseline_decode(sm, prompt, n_tokens):
    """The restated reference path on one host core (the reference runs m = 1 matmuls serially,
    parallel.rs:90-92): feeds at positions PROMPT.. after a prime."""
    from tests import oracle as O
    om = O.OracleModel(sm, threads=1)
    toks, _ = om.generate_greedy(prompt, 1)          # prime + first select, untimed
    t0 = time.perf_counter()
    tok = int(toks[0])
    for _ in range(n_tokens):
        p = om.feed(tok)
        tok = int(np.argmax(p))
    dt = time.perf_counter() - t0
    om.close()
    return n_tokens / dt


def cpu_baseline_score(sm, ids_row, threads):
    from tests import oracle as O
    om = O.OracleModel(sm, threads=threads)
    t0 = time.perf_counter()
    om.token_logprobs(ids_row, 1)
    dt = time.perf_counter() - t0
    om.close()
    return (len(ids_row) - 1) / dt


def cpu_baseline_llama(sml, prompt, n_tokens):
    """The restated LlamaModel::forward_one (llm.rs:610-618) on one host core: n_tokens cached steps
    after the prompt. Building the f32 model (1.04 G weights) is not timed."""
    from tests import oracle as O
    om = O.OracleLlama(sml, threads=1)
    logits = None
    for t in prompt:
        logits = om.forward_one(int(t))
    t0 = time.perf_counter()
    for _ in range(n_tokens):
        logits = om.forward_one(int(np.argmax(logits)))
    dt = time.perf_counter() - t0
    om.close()
    return n_tokens / dt


def run_reference(args, rank):
    """--impl reference: the CPU restatement of the reference path, bounded samples."""
    if rank != 0:
        return
    from ferrum_cpu_b200 import synth
    cores = os.cpu_count() or 1
    if args.workload == "llama-1b":
        sml = synth.llama_named("llama-1b", seed=0)
        n = 4
        v = cpu_baseline_llama(sml, synth.token_ids(0, 8, sml.dims["vocab"]), n)
        unit, metric = "tokens/s", "Q8_0 Llama-1B-shaped batch-1 greedy decode tokens/s"
        sample, used = f"{n} KV-cached steps after an 8-token prompt, 1 thread (f32 Linear with one row is serial in the reference)", 1
        cfg = {"workload": "Llama-3.2-1B shape: L16 d2048 H32 KV8 hd64 F8192 ctx2048 V32000, Q8_0", "sample": f"{n} tokens"}
        sm = None
    else:
        sm = synth.named("small", seed=0)
    if sm is None:
        pass
    elif args.workload == "score":
        ids = synth.token_ids(1, SEQ_LEN, sm.dims[5])
        vals = [cpu_baseline_score(sm, ids, cores) for _ in range(max(1, min(args.steps, 2)))]
        v, unit, metric = statistics.median(vals), "positions/s", "Q8_0 GPT-2-small log-likelihood positions/s"
        sample, used = f"one {SEQ_LEN}-id window of configs[2] per step, {cores} threads", cores
        cfg = {"workload": "configs[2] GPT-2-small Q8_0 scoring, 512 x 1024 ids", "sample": "1 window"}
    else:
        prompt = synth.token_ids(0, PROMPT, sm.dims[5])
        n = 8
        vals = [cpu_baseline_decode(sm, prompt, n) for _ in range(max(1, min(args.steps, 3)))]
        v, unit, metric = statistics.median(vals), "tokens/s", METRIC
        sample, used = f"{n} KV-cached feeds from position {PROMPT} of configs[1] per step, 1 thread (m=1 is serial in the reference)", 1
        cfg = {"workload": "configs[1] GPT-2-small Q8_0 decode, 32-token prompt, 256 greedy tokens", "sample": f"{n} tokens"}
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": v, "unit": unit, "cores": used, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", choices=["decode", "score", "both", "streams-medium", "llama-1b"], default="both",
                    help="both: configs[1] decode (+ 8 side-by-side streams) and configs[2] scoring; streams-medium: the decode "
                         "half of configs[4] on the GPT-2-medium shape (64 streams split over the ranks); llama-1b: greedy decode and "
                         "one-window scoring of a Llama-3.2-1B-shaped Q8_0 model (the imported-model path, replicas per rank)")
    ap.add_argument("--score-steps", type=int, default=2)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--score-math", choices=["bf16x3", "fp32"], default="bf16x3",
                    help="math mode of the scoring GEMMs: tcgen05 bf16 3-term split, or fp32 CUDA cores")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist

    import ferrum_cpu_b200 as fcb
    from ferrum_cpu_b200 import shard, synth

    if fcb.device_count() < 1:
        raise SystemExit("bench.py needs a B200: libferrum_cuda has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    hbm_peak, tf_peak, peak_kind = peaks()
    if args.workload == "streams-medium":
        # configs[4], decode half: 64 streams of 64-id prompts + 128 greedy tokens, split over the ranks
        smm = synth.named("medium", seed=0)
        gmm = fcb.CudaSlm(smm.config, smm.weights, device=local)
        a0, a1 = shard.shard_range(64, rank, world)
        prompts = np.stack([synth.token_ids(200 + i, 64, smm.dims[5]) for i in range(a0, a1)])
        gmm.decode_batch(prompts, 128)
        ms = []
        barrier()
        for _ in range(args.steps):
            gmm.decode_batch(prompts, 128)
            ms.append(gmm.last_batch_ms)
        barrier()
        step_ms = max_over_ranks(sum(ms) / len(ms))
        if rank == 0:
            print(json.dumps({"metric": "Q8_0 GPT-2-medium decode tokens/s, 64 concurrent streams (configs[4])", "value": 64 * 128 / (step_ms / 1e3),
                              "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "ms_per_step": step_ms, "higher_is_better": True,
                              "scaling": "strong", "dtype": "f32", "data": "synthetic",
                              "config": {"workload": "configs[4] decode: L24 d1024 H16 F4096 ctx1024 V50257, 64 streams x (64-id prompt + 128 greedy tokens), "
                                                     "%d streams per GPU, up to 8 side by side; prompts primed as one batch per wave; device time "
                                                     "includes the primes" % (a1 - a0)}}))
        gmm.close()
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "llama-1b":
        # The imported Llama / Qwen path (llm.rs) on a 1B-class shape: batch-1 greedy decode and window scoring.
        from ferrum_cpu_b200.engine import sampling
        from ferrum_cpu_b200.llama import CudaLlama
        sml = synth.llama_named("llama-1b", seed=0, math_mode=fcb.FC_MATH_BF16X3)
        c = sml.dims
        gml = CudaLlama.from_synth(sml, device=local)
        cache = gml.new_cache()
        prompt = synth.token_ids(rank, PROMPT, c["vocab"])
        greedy = sampling(temperature=0.0)
        for _ in range(args.warmup):
            gml.generate(prompt, NEW_TOKENS, greedy, cache=cache)
        fcb.take_launch_count()
        ms, wall = [], []
        barrier()
        for _ in range(args.steps):
            t0 = time.perf_counter()
            gml.generate(prompt, NEW_TOKENS, greedy, cache=cache)     # host ids in, host ids out
            wall.append(time.perf_counter() - t0)
            ms.append(cache.last_decode_ms)
        barrier()
        launches = fcb.take_launch_count()
        step_ms = max_over_ranks(sum(ms) / len(ms))
        wall_s = max_over_ranks(sum(wall) / len(wall))
        kvd = c["n_kv_head"] * c["head_dim"]
        kv_bytes = c["n_layer"] * 2 * (PROMPT + NEW_TOKENS / 2) * kvd * 4
        per_token = sml.q8_weight_bytes + kv_bytes + c["n_layer"] * 2 * c["d_model"] * 4
        T = 1024
        ids = synth.token_ids(100 + rank, 4 * T, c["vocab"]).reshape(4, T)
        gml.score_sequences(ids, batch_windows=4)
        sms_ = []
        for _ in range(max(1, args.score_steps)):
            gml.score_sequences(ids, batch_windows=4)
            sms_.append(gml.last_score_ms)
        score_ms = max_over_ranks(sum(sms_) / len(sms_))
        qd = c["n_head"] * c["head_dim"]
        flop_pos = 2 * sml.q8_weight_bytes * 32 / 34 + c["n_layer"] * 4 * qd * (T + 1) / 2
        if rank == 0:
            gbs = per_token * NEW_TOKENS / (step_ms / 1e3) / 1e9
            print(json.dumps({
                "metric": "Q8_0 Llama-1B-shaped batch-1 greedy decode tokens/s", "value": world * NEW_TOKENS / (step_ms / 1e3),
                "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "Llama-3.2-1B shape: L16 d2048 H32 KV8 hd64 F8192 ctx2048 V32000, Q8_0, %d-token prompt, %d greedy "
                                       "tokens, one replica per GPU; weights (1.1 GB) exceed the L2" % (PROMPT, NEW_TOKENS)},
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak, "traffic": None,
                             "peak_kind": peak_kind, "algorithmic_bytes_per_token": per_token},
                "e2e": {"value": world * NEW_TOKENS / wall_s, "unit": "tokens/s", "h2d_bytes_per_step": PROMPT * 4 + 8,
                        "d2h_bytes_per_step": NEW_TOKENS * 4 + 8 + 32, "note": "includes priming the prompt (one window forward)"},
                "gpu_launches": int(launches),
                "cpu_baseline": (None if args.no_cpu_baseline else
                                 {"value": cpu_baseline_llama(sml, synth.token_ids(0, 8, c["vocab"]), 4), "unit": "tokens/s", "cores": 1,
                                  "kind": "port", "sample": "4 KV-cached steps after an 8-token prompt, 1 thread"}),
                "scoring": {"value": world * 4 * T / (score_ms / 1e3), "unit": "positions/s", "ms_per_step": score_ms,
                            "tflops_algorithmic": flop_pos * 4 * T / (score_ms / 1e3) / 1e12,
                            "workload": "4 windows x 1024 ids, tcgen05 bf16x3 projections and grouped-query attention, exact log-softmax tail"}}))
        gml.close()
        if world > 1:
            dist.destroy_process_group()
        return
    # decode always runs fp32 FMA; the prefill GEMMs of scoring run the tensor-core math mode
    sm = synth.named("small", seed=0, math_mode=fcb.FC_MATH_FP32 if args.score_math == "fp32" else fcb.FC_MATH_BF16X3)
    dims = sm.dims
    V = dims[5]
    gm = fcb.CudaSlm(sm.config, sm.weights, device=local)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")   # > 126 MB L2
    out = {}

    if args.workload in ("decode", "both"):
        prompt = torch.from_numpy(synth.token_ids(rank, PROMPT, V).copy()).pin_memory()
        toks = torch.empty(NEW_TOKENS, dtype=torch.int32).pin_memory()
        pn, tn = prompt.numpy(), toks.numpy()
        for _ in range(max(3, args.warmup)):
            gm.generate_tokens(pn, NEW_TOKENS, out=tn)
        fcb.take_launch_count()
        sampler = ClockSampler(local) if rank == 0 else None
        dev_ms, wall = [], []
        barrier()
        t_all0 = time.perf_counter()
        for _ in range(args.steps):
            flush.zero_()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            gm.generate_tokens(pn, NEW_TOKENS, out=tn)   # H2D prompt, prime, 256 feeds, D2H tokens
            wall.append(time.perf_counter() - t0)
            dev_ms.append(gm.last_decode_ms)
        barrier()
        t_all = time.perf_counter() - t_all0
        clocks = sampler.stop() if sampler else None
        launches = fcb.take_launch_count()
        step_ms = max_over_ranks(sum(dev_ms) / len(dev_ms))
        e2e_s = max_over_ranks(sum(wall) / len(wall))
        tok_s = world * NEW_TOKENS / (step_ms / 1e3)
        bpt = decode_bytes_per_token(dims, PROMPT, NEW_TOKENS)
        achieved = bpt * (NEW_TOKENS / (step_ms / 1e3)) / 1e9
        out = {
            "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "configs[1] GPT-2-small Q8_0 decode: L12 d768 H12 F3072 ctx1024 V50257, batch 1, "
                                   "32-token prompt, 256 greedy tokens, KV cache; one independent stream per GPU (replicas only)",
                       "l2": "256 MiB buffer written between steps; 143.6 MB streamed per token exceeds the 126 MB L2",
                       "timed_region": "the 256 feeds after the prime (CUDA events on the launching stream)",
                       "wall_s_all_steps": t_all},
            "e2e": {"value": world * NEW_TOKENS / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": PROMPT * 4,
                    "d2h_bytes_per_step": NEW_TOKENS * 4 + 32,
                    "note": "fc_generate_greedy from pinned host buffers: prompt upload, 32-token prime, 256 feeds, token download"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "traffic": DECODE_DRAM_BYTES_PER_TOKEN * 32, "peak_kind": peak_kind,
                         "what": "decode_mega_kernel, launches of 32 tokens: %.1f MB algorithmic per token; traffic = "
                                 "ncu dram read+write of a one-token launch at position 38 (134.8 + 4.98 MB, "
                                 "profiles/decode_mega_kernel_gpt2small_7tokens.md) scaled to 32 tokens" % (bpt / 1e6)},
            "clocks": clocks,
        }
        # the per-GPU share of configs[4]'s 64 streams (8 at 8 GPUs), on this model: side-by-side persistent kernels
        sp = np.stack([synth.token_ids(200 + 8 * rank + i, 64, V) for i in range(8)])
        gm.decode_batch(sp, 128)
        ms = []
        barrier()
        for _ in range(3):
            gm.decode_batch(sp, 128)
            ms.append(gm.last_batch_ms)
        barrier()
        sb_ms = max_over_ranks(sum(ms) / len(ms))
        out["decode_streams"] = {"metric": "Q8_0 GPT-2-small decode tokens/s, 8 concurrent streams per GPU", "value": world * 8 * 128 / (sb_ms / 1e3),
                                 "unit": "tokens/s", "ms_per_step": sb_ms, "n_gpus": world,
                                 "config": {"workload": "8 streams per GPU x (64-id prompt + 128 greedy tokens), one persistent kernel per stream on "
                                                        "an eighth of the SMs; device time includes the batched prime of the 8 prompts"},
                                 "gpu_launches": int(fcb.take_launch_count())}

    if args.workload in ("score", "both"):
        ids_all = synth.token_ids(1, N_SEQ * SEQ_LEN, V).reshape(N_SEQ, SEQ_LEN)
        first, last = shard.shard_range(N_SEQ, rank, world)      # contiguous block of sequences per rank
        per = last - first
        mine = torch.from_numpy(ids_all[first:last].copy()).pin_memory()
        lp = torch.empty((per, SEQ_LEN), dtype=torch.float32).pin_memory()
        bw = 64
        gm.score_sequences(mine.numpy()[:bw], batch_windows=bw, lp_out=lp.numpy()[:bw])   # warm-up (allocates the workspace)
        if world > 1:   # warm-up of the gather too: NCCL opens its peer channels on the first send
            shard.gather_rows(lp.numpy(), N_SEQ, rank, world, device=torch.device("cuda", local))
            torch.cuda.synchronize()
        fcb.take_launch_count()
        dev_ms, wall = [], []
        barrier()
        for _ in range(args.score_steps):
            flush.zero_()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            scores, _ = gm.score_sequences(mine.numpy(), batch_windows=bw, lp_out=lp.numpy())
            if world > 1:   # the one collective of the path: gather the per-token log-probs to rank 0
                shard.gather_rows(lp.numpy(), N_SEQ, rank, world, device=torch.device("cuda", local))
                torch.cuda.synchronize()
            wall.append(time.perf_counter() - t0)
            dev_ms.append(gm.last_score_ms)
        barrier()
        s_launch = fcb.take_launch_count()
        step_ms = max_over_ranks(sum(dev_ms) / len(dev_ms))
        e2e_s = max_over_ranks(sum(wall) / len(wall))
        positions = N_SEQ * SEQ_LEN
        fl = score_flops_per_position(dims) * positions
        score = {
            "metric": "Q8_0 GPT-2-small log-likelihood positions/s", "value": positions / (step_ms / 1e3), "unit": "positions/s",
            "n_gpus": world, "steps": args.score_steps, "ms_per_step": step_ms, "scaling": "strong" if world > 1 else "n/a",
            "config": {"workload": "configs[2]: %d sequences x %d ids, full-window prefill, per-token log-probs, %d windows per forward"
                       % (N_SEQ, SEQ_LEN, bw),
                       "math": "linear layers: tcgen05 kind::f16, bf16 3-term split of f32 operands, fp32 TMEM accumulate"
                               if args.score_math == "bf16x3" else "fp32 CUDA cores"},
            "dtype": "bf16x3" if args.score_math == "bf16x3" else "f32",
            "e2e": {"value": positions / e2e_s, "unit": "positions/s", "h2d_bytes_per_step": per * SEQ_LEN * 4,
                    "d2h_bytes_per_step": per * SEQ_LEN * 4 + per * 24},
            "gpu_launches": int(s_launch),
            # per GPU: every rank runs the same kernels on its own block of sequences
            "roofline": {"bound": "tensor", "achieved": fl / world / (step_ms / 1e3) / 1e12, "peak": tf_peak, "unit": "TFLOP/s",
                         "frac": fl / world / (step_ms / 1e3) / 1e12 / tf_peak, "traffic": None, "peak_kind": peak_kind,
                         "what": "per GPU: algorithmic FLOP of the rank's sequences / its step time"},
            "checksum_logprob": sum_over_ranks(float(sum(s.logprob for s in scores))),
        }
        if out:
            out["score"] = score
        else:
            out = dict(score, warmup=1, higher_is_better=True, vs_baseline=None, dtype="f32", data="synthetic")

    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            if "tokens/s" == out.get("unit"):
                n = 16
                v = cpu_baseline_decode(sm, synth.token_ids(0, PROMPT, V), n)
                out["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": 1, "kind": "port",
                                       "sample": f"{n} KV-cached feeds from position {PROMPT} of configs[1]; 1 thread because the "
                                                 f"reference runs m=1 matmuls serially; host has {os.cpu_count()} cores"}
            if "score" in out or out.get("unit") == "positions/s":
                cores = os.cpu_count() or 1
                v = cpu_baseline_score(sm, synth.token_ids(1, SEQ_LEN, V), cores)
                tgt = out["score"] if "score" in out else out
                tgt["cpu_baseline"] = {"value": v, "unit": "positions/s", "cores": cores, "kind": "port",
                                       "sample": f"one {SEQ_LEN}-id window of configs[2], {cores} threads"}
        print(json.dumps(out))
    gm.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
