#!/usr/bin/env python
"""Benchmark of the Q8_0 GPT-2 forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload ...] [--impl ours|reference]
    python bench.py --case decode|score|linear|rowq|ggml-linear|streams|llama-decode|llama-score [...]

Workloads (synthetic, seeded; shapes of the reference's configurations):
  decode        : GPT-2-small-shaped Q8_0 model, batch 1, 32-token prompt, 256 greedy tokens with a
                  KV cache. One step = one such generation. metric: decode tokens/s. At N GPUs every
                  rank decodes its own stream (replicas only; the path does not shard).
  score         : the same model, 512 sequences x 1024 ids scored per step (per-token log-probs),
                  sharded by sequence over the ranks with one gather of the results.
  both (default): decode + score, plus the concurrent-stream decodes (8 streams on the small shape,
                  64 streams on the GPT-2-medium shape, split over the ranks); a short `summary`
                  object closes the line.
  streams-medium: the decode half of the medium-shaped configuration alone.
  score-medium  : its scoring half, 1024 sequences x 1024 ids split over the ranks.
  sweep         : the five (M, K, N) shapes of the standalone Q8_0 matmul sweep, each against the
                  oracle's matmul engine.
  tiny          : the 4-block CPU-sized configuration (16-token prompt, 64 greedy tokens).
  llama-1b      : the imported Llama-shaped decoder.

--case runs one small, self-terminating piece of the same kernels (a few tokens / windows / one
product) and prints CUDA-event times: these are the command lines the profiler notes under
profiles/ were captured with.

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


def decode_dram_bytes_per_token():
    """dram__bytes_read.sum + dram__bytes_write.sum of the persistent decode kernel per token, from the
    tracked capture record (which names the kernel revision it was taken at); None when absent."""
    path = os.path.join(ROOT, "profiles", "decode_mega_kernel_traffic.json")
    if not os.path.exists(path):
        return None
    rec = json.load(open(path))
    return float(rec["dram_bytes_read_per_token"]) + float(rec["dram_bytes_write_per_token"])


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


SWEEP_SHAPES = [(1, 768, 2304), (1, 3072, 768), (1, 768, 50257), (512, 768, 3072), (4096, 1024, 4096)]
STREAM_PROMPT, STREAM_NEW, STREAM_SEED = 64, 128, 200


def stream_bytes_per_step(dims, S, p_first, n_steps):
    """Algorithmic HBM bytes of one lock-step decode step for S streams, averaged over the cache positions
    p_first .. p_first + n_steps - 1: every Q8_0 matrix once, the f32 vectors once, and per stream one
    position row, one token row and the f32 K / V rows of positions 0..p (read) and p (written)."""
    L, d, H, F, T, V = dims
    q8 = (L * (4 * d * d + 2 * d * F) + d * V) * 34 // 32
    small = (L * (9 * d + F) + 2 * d) * 4
    per_stream = d * 4 + d * 34 // 32
    kv = sum(L * 2 * (p + 1) * d * 4 + L * 2 * d * 4 for p in range(p_first, p_first + n_steps)) / max(n_steps, 1)
    return q8 + small + S * (per_stream + kv)


def run_streams(fcb, synth, shard, name, n_streams, local, rank, world, steps, barrier, max_over_ranks, hbm_peak, peak_kind):
    """The concurrent-stream decode workload on model `name`: n_streams streams (split over the ranks in
    contiguous blocks) x (64-id prompt + 128 greedy tokens), lock step. Returns the result object."""
    sm = synth.named(name, seed=0, math_mode=fcb.FC_MATH_BF16X3)
    gm = fcb.CudaSlm(sm.config, sm.weights, device=local)
    a0, a1 = shard.shard_range(n_streams, rank, world)
    S = a1 - a0
    prompts = np.stack([synth.token_ids(STREAM_SEED + i, STREAM_PROMPT, sm.dims[5]) for i in range(a0, a1)])
    outs = gm.decode_batch(prompts, STREAM_NEW)                # warm-up: builds the weight copies, caches and the step graph
    fcb.take_launch_count()
    ms, prime, wall = [], [], []
    barrier()
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        outs = gm.decode_batch(prompts, STREAM_NEW)            # host prompts in, host tokens out
        wall.append(time.perf_counter() - t0)
        ms.append(gm.last_batch_ms)
        prime.append(gm.last_batch_prime_ms)
    barrier()
    launches = fcb.take_launch_count()
    step_ms = max_over_ranks(sum(ms) / len(ms))
    prime_ms = max_over_ranks(sum(prime) / len(prime))
    wall_s = max_over_ranks(sum(wall) / len(wall))
    n_steps = STREAM_NEW - 1                                    # token 1 comes out of the prime
    per_step_s = (step_ms - prime_ms) / 1e3 / n_steps
    byts = stream_bytes_per_step(sm.dims, S, STREAM_PROMPT, n_steps)
    gbs = byts / per_step_s / 1e9
    checksum = int(sum(int(o.sum()) for o in outs))
    gm.close()
    return {
        "metric": "Q8_0 GPT-2-%s decode tokens/s, %d concurrent streams" % (name, n_streams),
        "value": n_streams * STREAM_NEW / (step_ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": max(1, steps),
        "ms_per_step": step_ms, "prime_ms": prime_ms, "us_per_decode_step": per_step_s * 1e6,
        "higher_is_better": True, "scaling": "strong" if world > 1 else "n/a", "dtype": "f32", "data": "synthetic",
        "config": {"workload": "%d streams x (%d-id prompt + %d greedy tokens) on the GPT-2-%s shape, %d streams per GPU in lock "
                               "step: one tensor-core window forward primes all prompts, then every step reads each Q8_0 matrix "
                               "once for all streams; device time includes the primes" % (n_streams, STREAM_PROMPT, STREAM_NEW, name, S)},
        "e2e": {"value": n_streams * STREAM_NEW / wall_s, "unit": "tokens/s", "h2d_bytes_per_step": S * STREAM_PROMPT * 4,
                "d2h_bytes_per_step": S * STREAM_NEW * 4 + S * 4},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak, "traffic": None,
                     "peak_kind": peak_kind,
                     "what": "per GPU, decode steps only (prime excluded): %.1f MB algorithmic per step for %d streams "
                             "(weights once + f32 K/V rows per stream)" % (byts / 1e6, S)},
        "token_checksum": checksum,
    }


def run_sweep(fcb, synth, torch, shapes, reps, with_oracle):
    """The standalone Q8_0 matmul sweep: device time of one product with the weight resident (CUDA events on
    the launching stream, L2 flushed between repetitions), and the error against the oracle's matmul engine."""
    import ctypes as C
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rows = []
    for (m, k, n) in shapes:
        w = synth.Rng(21).normal(n * k, 0.02)
        wq = synth.q8_0_quantize(w)
        x_h = synth.Rng(22).normal(m * k, 1.0).reshape(m, k)
        qw = fcb.QWeight(wq, n, k)
        x = torch.from_numpy(x_h).cuda()
        y = torch.empty(m, n, device="cuda")
        want = None
        if with_oracle:
            from tests import oracle as O
            want = O.linear(x_h, O.expand_kn(wq, n, k), None, threads=os.cpu_count() or 1)
        byts = n * k * 34 / 32 + 4 * m * k + 4 * m * n
        row = {"M": m, "K": k, "N": n, "algorithmic_bytes": byts, "flop": 2.0 * m * k * n}
        for mode, label in ((fcb.FC_MATH_FP32, "fp32"), (fcb.FC_MATH_BF16X3, "bf16x3")):
            if m == 1 and mode != fcb.FC_MATH_FP32:
                continue                                   # one row is the decode GEMV whatever the mode
            best = None
            for _ in range(max(3, reps)):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                qw.linear_dev(x.data_ptr(), None, y.data_ptr(), m, mode, st)
                e1.record()
                torch.cuda.synchronize()
                t = e0.elapsed_time(e1)
                best = t if best is None else min(best, t)
            r = {"us": best * 1e3, "GBps": byts / best / 1e6, "TFLOPs": 2.0 * m * k * n / best / 1e9}
            if want is not None:
                got = y.cpu().numpy()
                r["max_abs_err"] = float(np.abs(got - want).max())
                r["max_err_rel_to_scale"] = float(np.abs(got - want).max() / np.abs(want).max())
            row["gemv" if m == 1 else label] = r
        qw.close()
        rows.append(row)
    return rows


def run_case(a):
    """Small self-terminating cases for profiler captures (same kernels as the workloads)."""
    import ctypes as C

    import torch

    import ferrum_cpu_b200 as fcb
    from ferrum_cpu_b200 import synth
    if a.case == "linear":
        for row in run_sweep(fcb, synth, torch, [(a.m, a.k, a.n)], a.reps, False):
            print(json.dumps(row))
        return
    if a.case == "rowq":
        from ferrum_cpu_b200.engine import RowQWeight
        w = synth.Rng(21).normal(a.k * a.n, 0.02).reshape(a.k, a.n)
        qw = RowQWeight.from_f32(w, a.kind)
        x = torch.randn(a.m, a.k, device="cuda")
        bias = torch.zeros(a.n, device="cuda")
        y = torch.empty(a.m, a.n, device="cuda")
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        st = torch.cuda.current_stream().cuda_stream
        for _ in range(a.reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            qw.linear_dev(x.data_ptr(), bias.data_ptr(), y.data_ptr(), a.m, C.c_void_p(st))
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            byts = a.k * a.n / (2 if a.kind else 1) + 4 * a.k + 4 * a.m * (a.k + a.n)
            print(f"rowq {'int4' if a.kind else 'int8'} M={a.m} K={a.k} N={a.n}: {ms * 1e3:.1f} us, {byts / ms / 1e6:.1f} GB/s")
        return
    if a.case == "ggml-linear":
        # one matrix kept in a ggml block format (--native: ggml type), decoded inside the product
        import numpy as np
        from ferrum_cpu_b200 import _lib
        t = a.native if a.native >= 0 else 12
        vals, bb = {2: (32, 18), 6: (32, 22), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210)}[t]
        rng = np.random.default_rng(0)
        raw = rng.integers(0, 256, size=(a.n * a.k // vals, bb), dtype=np.uint8)
        for at in {2: [0], 6: [0], 8: [0], 12: [0, 2], 13: [0, 2], 14: [208]}[t]:
            raw[:, at:at + 2] = (rng.standard_normal(raw.shape[0]) * 0.01).astype(np.float16).view(np.uint8).reshape(-1, 2)
        h = C.c_void_p()
        rc = _lib.lib().fc_ggml_weight_upload(0, t, raw.ctypes.data_as(C.c_void_p), raw.size, a.n, a.k, C.byref(h))
        assert rc == 0, rc
        x = torch.randn(a.m, a.k, device="cuda")
        y = torch.empty(a.m, a.n, device="cuda")
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        st = torch.cuda.current_stream().cuda_stream
        for _ in range(a.reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _lib.lib().fc_ggml_linear_dev(h, C.c_void_p(x.data_ptr()), None, C.c_void_p(y.data_ptr()), a.m, C.c_void_p(st))
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            byts = raw.size + 4 * a.m * (a.k + a.n)
            print(f"ggml type {t} M={a.m} K={a.k} N={a.n}: {ms * 1e3:.1f} us, {byts / ms / 1e6:.1f} GB/s")
        _lib.lib().fc_ggml_weight_free(h)
        return
    if a.case.startswith("llama"):
        from ferrum_cpu_b200.engine import sampling
        from ferrum_cpu_b200.llama import CudaLlama
        name = a.model if a.model.startswith("llama") else "llama-1b"
        sm = synth.llama_named(name, seed=0, math_mode=a.math)
        c = sm.dims
        if a.native >= 0:
            # every matrix as random blocks of one ggml type in a temporary GGUF file, kept in that format on the device
            import tempfile
            import numpy as np
            from ferrum_cpu_b200 import gguf_file
            vals, bb = {2: (32, 18), 6: (32, 22), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210)}[a.native]
            rng = np.random.default_rng(0)

            def blocks(n):
                raw = rng.integers(0, 256, size=(n // vals, bb), dtype=np.uint8)
                for at in {2: [0], 6: [0], 8: [0], 12: [0, 2], 13: [0, 2], 14: [208]}[a.native]:
                    raw[:, at:at + 2] = (rng.standard_normal(n // vals) * 0.01).astype(np.float16).view(np.uint8).reshape(-1, 2)
                return raw.reshape(-1)
            c = sm.dims
            d, F, qd, kvd = c["d_model"], c["d_ff"], c["n_head"] * c["head_dim"], c["n_kv_head"] * c["head_dim"]
            shapes = {"attn_q": qd * d, "attn_k": kvd * d, "attn_v": kvd * d, "attn_output": d * qd, "ffn_gate": F * d, "ffn_up": F * d,
                      "ffn_down": d * F}
            raw = {f"blk.{i}.{stem}.weight": (a.native, blocks(n)) for i in range(c["n_layer"]) for stem, n in shapes.items()}
            raw["token_embd.weight"] = (a.native, blocks(c["vocab"] * d))
            tmp = tempfile.TemporaryDirectory()
            path = gguf_file.write_llama_gguf(os.path.join(tmp.name, "m.gguf"), sm, raw=raw)
            gm = CudaLlama.from_gguf(path, prec="native")
            name += f" native ggml type {a.native}"
            weight_bytes = sum(v[1].size for v in raw.values())   # the tied head is the embedding table, read once per token
        else:
            gm = CudaLlama.from_synth(sm, prec=None if a.packed < 0 else a.packed)
            weight_bytes = sm.q8_weight_bytes
        if a.packed >= 0:
            name += " packed int4" if a.packed else " packed int8"
        if a.case == "llama-decode":
            prompt = synth.token_ids(0, a.prompt, c["vocab"])
            cache = gm.new_cache()
            kvd = c["n_kv_head"] * c["head_dim"]
            for _ in range(a.reps):
                gm.generate(prompt, a.tokens, sampling(temperature=0.0), cache=cache)
                us = cache.last_decode_ms / a.tokens * 1e3
                kv = c["n_layer"] * 2 * (a.prompt + a.tokens / 2) * kvd * 4
                print(f"{name} decode {a.tokens} tokens: device {us:.1f} us/token, {(weight_bytes + kv) / us / 1e3:.0f} GB/s "
                      f"algorithmic, launches {fcb.take_launch_count()}")
        else:
            T = min(c["ctx"], 1024)
            ids = synth.token_ids(1, a.windows * T, c["vocab"]).reshape(a.windows, T)
            for _ in range(a.reps):
                gm.score_sequences(ids, batch_windows=a.windows)
                print(f"{name} score {a.windows} x {T}: device {gm.last_score_ms:.2f} ms, launches {fcb.take_launch_count()}")
        gm.close()
        return
    sm = synth.named(a.model, seed=0, math_mode=a.math)
    V, T = sm.dims[5], sm.dims[4]
    gm = fcb.CudaSlm(sm.config, sm.weights)
    if a.case == "decode":
        prompt = synth.token_ids(0, a.prompt, V)
        gm.set_decode_mode(a.mode)
        for _ in range(a.reps):
            gm.generate_tokens(prompt, a.tokens)
            print(f"decode {a.tokens} tokens: device {gm.last_decode_ms / a.tokens * 1e3:.1f} us/token, launches {fcb.take_launch_count()}")
        if a.trace and a.mode == 0:
            # phase timeline of one token of the persistent kernel (CTA 0), mean over blocks
            gm.set_trace(True)
            gm.generate_tokens(prompt, a.tokens)
            t = gm.read_trace()
            gm.set_trace(False)
            L = sm.dims[0]
            names = ["ln1", "qkv", "barrier", "attn", "barrier", "combine", "out", "barrier", "load+ln2", "up", "barrier", "load",
                     "down", "barrier", "load"]
            if len(t) >= 1 + 15 * L:
                per = np.diff(t[:1 + 15 * L]).reshape(L, 15)
                print("phase timeline of CTA 0 (ns, mean over blocks): " + ", ".join(f"{n} {per[:, i].mean():.0f}" for i, n in enumerate(names)))
                print(f"blocks {per.sum():.0f} ns; head + select {t[-1] - t[15 * L]:.0f} ns; token {t[-1]:.0f} ns")
    elif a.case == "streams":
        prompts = np.stack([synth.token_ids(STREAM_SEED + i, a.prompt, V) for i in range(a.streams)])
        for _ in range(a.reps):
            gm.decode_batch(prompts, a.tokens)
            print(f"{a.streams} streams x {a.tokens} tokens: device {gm.last_batch_ms:.3f} ms (prime {gm.last_batch_prime_ms:.3f} ms), "
                  f"launches {fcb.take_launch_count()}")
    else:
        ids = synth.token_ids(1, a.windows * T, V).reshape(a.windows, T)
        for _ in range(a.reps):
            gm.score_sequences(ids, batch_windows=a.windows)
            print(f"score {a.windows} x {T}: device {gm.last_score_ms:.2f} ms, launches {fcb.take_launch_count()}")
    gm.close()


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
    ap.add_argument("--workload", choices=["decode", "score", "both", "streams-medium", "score-medium", "sweep", "tiny", "llama-1b"],
                    default="both", help="see the module docstring")
    ap.add_argument("--case", choices=["decode", "score", "linear", "rowq", "ggml-linear", "streams", "llama-decode", "llama-score"], default=None,
                    help="run one small self-terminating case (for profiler captures) instead of a workload")
    ap.add_argument("--model", default="small")
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=32)
    ap.add_argument("--windows", type=int, default=4)
    ap.add_argument("--streams", type=int, default=8)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--n", type=int, default=50257)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--math", type=int, default=0, help="--case: 0 fp32 CUDA cores, 1 tcgen05 bf16x3")
    ap.add_argument("--kind", type=int, default=0, help="--case rowq: 0 int8, 1 int4")
    ap.add_argument("--native", type=int, default=-1, help="--case llama-*: matrices kept in this ggml block format (2 Q4_0, 6 Q5_0, 8 Q8_0, 12 Q4_K, 13 Q5_K, 14 Q6_K) and decoded in the kernels")
    ap.add_argument("--packed", type=int, default=-1, help="--case llama-*: every Linear packed to per-row int8 (0) / int4 (1), as the reference's importer does")
    ap.add_argument("--mode", type=int, default=0, help="--case decode: 0 persistent kernel, 1 one kernel per operation")
    ap.add_argument("--trace", action="store_true", help="--case decode: print the phase timeline of one token")
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
    if args.case:
        run_case(args)
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
        # the decode half of the medium-shaped configuration: 64 streams split over the ranks
        res = run_streams(fcb, synth, shard, "medium", 64, local, rank, world, args.steps, barrier, max_over_ranks, hbm_peak, peak_kind)
        if rank == 0:
            print(json.dumps(dict(res, warmup=1, vs_baseline=None)))
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "score-medium":
        # its scoring half: 1024 sequences x 1024 ids, split over the ranks in contiguous blocks
        smm = synth.named("medium", seed=0, math_mode=fcb.FC_MATH_BF16X3)
        gmm = fcb.CudaSlm(smm.config, smm.weights, device=local)
        n_seq = 1024
        a0, a1 = shard.shard_range(n_seq, rank, world)
        ids = synth.token_ids(1, n_seq * SEQ_LEN, smm.dims[5]).reshape(n_seq, SEQ_LEN)[a0:a1]
        gmm.score_sequences(ids[:32], batch_windows=32)
        ms, wall = [], []
        barrier()
        for _ in range(max(1, args.score_steps)):
            t0 = time.perf_counter()
            scores, _ = gmm.score_sequences(ids, batch_windows=32)
            wall.append(time.perf_counter() - t0)
            ms.append(gmm.last_score_ms)
        barrier()
        step_ms = max_over_ranks(sum(ms) / len(ms))
        wall_s = max_over_ranks(sum(wall) / len(wall))
        fl = score_flops_per_position(smm.dims) * n_seq * SEQ_LEN
        tf = fl / world / (step_ms / 1e3) / 1e12
        checksum = sum_over_ranks(float(sum(sc.logprob for sc in scores)))   # a collective: every rank takes part
        if rank == 0:
            print(json.dumps({
                "metric": "Q8_0 GPT-2-medium log-likelihood positions/s", "value": n_seq * SEQ_LEN / (step_ms / 1e3), "unit": "positions/s",
                "n_gpus": world, "steps": max(1, args.score_steps), "warmup": 1, "ms_per_step": step_ms, "higher_is_better": True,
                "scaling": "strong" if world > 1 else "n/a", "vs_baseline": None, "dtype": "bf16x3", "data": "synthetic",
                "config": {"workload": "GPT-2-medium shape L24 d1024 H16 F4096 ctx1024 V50257: %d sequences x %d ids, full-window "
                                       "prefill, per-token log-probs, 32 windows per forward, %d sequences per GPU" % (n_seq, SEQ_LEN, a1 - a0)},
                "e2e": {"value": n_seq * SEQ_LEN / wall_s, "unit": "positions/s", "h2d_bytes_per_step": (a1 - a0) * SEQ_LEN * 4,
                        "d2h_bytes_per_step": (a1 - a0) * SEQ_LEN * 4},
                "roofline": {"bound": "tensor", "achieved": tf, "peak": tf_peak, "unit": "TFLOP/s", "frac": tf / tf_peak, "traffic": None,
                             "peak_kind": peak_kind, "what": "per GPU: algorithmic FLOP of the rank's sequences / its step time"},
                "checksum_logprob": checksum}))
        gmm.close()
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "sweep":
        rows = run_sweep(fcb, synth, torch, SWEEP_SHAPES, args.steps, rank == 0 and not args.no_cpu_baseline) if rank == 0 else []
        if rank == 0:
            big = rows[-1]
            print(json.dumps({
                "metric": "Q8_0 matmul sweep, (4096, 1024, 4096) TFLOP/s (bf16x3)", "value": big["bf16x3"]["TFLOPs"], "unit": "TFLOP/s",
                "n_gpus": 1, "steps": max(3, args.steps), "warmup": 0, "ms_per_step": big["bf16x3"]["us"] / 1e3, "higher_is_better": True,
                "scaling": "n/a", "vs_baseline": None, "dtype": "bf16x3 / f32", "data": "synthetic",
                "config": {"workload": "standalone Q8_0 linear, weight resident, five (M, K, N) shapes; M = 1 is the decode GEMV "
                                       "(GB/s of algorithmic bytes), M >= 512 the prefill GEMM in both math modes (TFLOP/s); 256 MiB "
                                       "written between repetitions; best of the repetitions; errors against the oracle's matmul engine"},
                "peaks": {"hbm_gbs": hbm_peak, "bf16_tflops": tf_peak, "kind": peak_kind},
                "shapes": rows}))
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "tiny":
        # the 4-block configuration the reference itself runs on a CPU: 16-token prompt, 64 greedy tokens
        smt = synth.named("tiny", seed=0)
        gmt = fcb.CudaSlm(smt.config, smt.weights, device=local)
        prompt = synth.token_ids(0, 16, smt.dims[5])
        for _ in range(max(3, args.warmup)):
            gmt.generate_tokens(prompt, 64)
        ms, wall = [], []
        barrier()
        for _ in range(args.steps):
            t0 = time.perf_counter()
            gmt.generate_tokens(prompt, 64)
            wall.append(time.perf_counter() - t0)
            ms.append(gmt.last_decode_ms)
        barrier()
        step_ms = max_over_ranks(sum(ms) / len(ms))
        wall_s = max_over_ranks(sum(wall) / len(wall))
        if rank == 0:
            res = {"metric": "Q8_0 tiny GPT-2 decode tokens/s (batch 1, KV cache, greedy)", "value": world * 64 / (step_ms / 1e3),
                   "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": step_ms,
                   "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                   "config": {"workload": "L4 d128 H4 F512 ctx128 V4096, 16-token prompt, 64 greedy tokens, one stream per GPU; the "
                                          "model (1.4 MB of Q8_0) lives in L2: latency-bound, no roofline"},
                   "e2e": {"value": world * 64 / wall_s, "unit": "tokens/s", "h2d_bytes_per_step": 64, "d2h_bytes_per_step": 64 * 4 + 32}}
            if not args.no_cpu_baseline and world == 1:
                res["cpu_baseline"] = {"value": cpu_baseline_decode(smt, prompt, 48), "unit": "tokens/s", "cores": 1, "kind": "port",
                                       "sample": "48 KV-cached feeds after the 16-token prompt, 1 thread"}
            print(json.dumps(res))
        gmt.close()
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
                         "traffic": None if decode_dram_bytes_per_token() is None else decode_dram_bytes_per_token() * 32,
                         "peak_kind": peak_kind,
                         "what": "decode_mega_kernel, launches of 32 tokens: %.1f MB algorithmic per token; traffic = ncu dram "
                                 "read + write of a one-token launch at position 38, scaled to 32 tokens" % (bpt / 1e6)},
            "clocks": clocks,
        }
        if args.workload == "both":
            # concurrent streams: 8 per GPU on this shape, and the medium-shaped 64-stream workload split over the ranks
            gm.close()
            gm = None
            out["decode_streams"] = run_streams(fcb, synth, shard, "small", 8 * world, local, rank, world, 3, barrier, max_over_ranks,
                                                hbm_peak, peak_kind)
            out["streams_medium"] = run_streams(fcb, synth, shard, "medium", 64, local, rank, world, 2, barrier, max_over_ranks,
                                                hbm_peak, peak_kind)
            gm = fcb.CudaSlm(sm.config, sm.weights, device=local)

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
        # the figures every reader needs, short and last (a log tail keeps them); at N > 1 the long descriptions go
        subs = [k for k in ("decode_streams", "streams_medium", "score") if k in out]
        if world > 1:
            for k in subs:
                out[k].pop("config", None)
                out[k].get("roofline", {}).pop("what", None)
        summary = {"n_gpus": world}
        if out.get("unit") == "tokens/s":
            summary.update(decode_tok_s=round(out["value"], 1), decode_e2e_tok_s=round(out["e2e"]["value"], 1),
                           decode_hbm_frac=round(out["roofline"]["frac"], 4))
        for k, short in (("decode_streams", "streams_small"), ("streams_medium", "streams_medium")):
            if k in out:
                summary[short + "_tok_s"] = round(out[k]["value"], 1)
                summary[short + "_e2e_tok_s"] = round(out[k]["e2e"]["value"], 1)
                summary[short + "_step_hbm_frac"] = round(out[k]["roofline"]["frac"], 4)
        sc = out.get("score", out if out.get("unit") == "positions/s" else None)
        if sc:
            summary.update(score_pos_s=round(sc["value"], 1), score_e2e_pos_s=round(sc["e2e"]["value"], 1), score_ms=round(sc["ms_per_step"], 2),
                           score_tensor_frac=round(sc["roofline"]["frac"], 4))
        out["summary"] = summary
        print(json.dumps(out))
    if gm is not None:
        gm.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
