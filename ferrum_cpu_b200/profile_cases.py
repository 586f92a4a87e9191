"""Small, self-terminating cases of the hot path for `ncu` captures.

    python -m ferrum_cpu_b200.profile_cases decode [--tokens 8] [--model small]
    python -m ferrum_cpu_b200.profile_cases score  [--windows 4] [--model small]
    python -m ferrum_cpu_b200.profile_cases linear --m 1 --k 768 --n 50257 [--reps 3]
    python -m ferrum_cpu_b200.profile_cases rowq --m 1 --k 2048 --n 8192 --kind 1 [--reps 3]
    python -m ferrum_cpu_b200.profile_cases llama-decode [--model llama-1b] [--tokens 64]
    python -m ferrum_cpu_b200.profile_cases llama-score  [--model llama-1b] [--windows 2] [--math 1]

Each case runs the same kernels as the benchmark on the same seeded synthetic model, but on a
few tokens / windows so that a multi-pass capture ends by itself. Prints CUDA-event times.
"""
import argparse
import ctypes as C
import time

import numpy as np

import ferrum_cpu_b200 as fcb
from ferrum_cpu_b200 import synth


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["decode", "score", "linear", "rowq", "llama-decode", "llama-score"])
    ap.add_argument("--model", default="small")
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=32)
    ap.add_argument("--windows", type=int, default=4)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--n", type=int, default=50257)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--math", type=int, default=0)
    ap.add_argument("--kind", type=int, default=0, help="rowq: 0 int8, 1 int4")
    ap.add_argument("--trace", action="store_true", help="decode: print the phase timeline of one token")
    ap.add_argument("--mode", type=int, default=0, help="decode: 0 persistent kernel, 1 one kernel per operation")
    a = ap.parse_args()
    if a.case == "linear":
        import torch
        w = synth.Rng(21).normal(a.n * a.k, 0.02)
        qw = fcb.QWeight(synth.q8_0_quantize(w), a.n, a.k)
        x = torch.randn(a.m, a.k, device="cuda")
        y = torch.empty(a.m, a.n, device="cuda")
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        st = torch.cuda.current_stream().cuda_stream
        for i in range(a.reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            qw.linear_dev(x.data_ptr(), None, y.data_ptr(), a.m, a.math, C.c_void_p(st))
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            byts = a.n * a.k * 34 / 32 + 4 * a.m * a.k + 4 * a.m * a.n
            print(f"linear M={a.m} K={a.k} N={a.n}: {ms * 1e3:.1f} us, {byts / ms / 1e6:.1f} GB/s, "
                  f"{2 * a.m * a.k * a.n / ms / 1e9:.2f} TFLOP/s")
        return
    if a.case == "rowq":
        import torch
        from ferrum_cpu_b200.engine import RowQWeight
        w = synth.Rng(21).normal(a.k * a.n, 0.02).reshape(a.k, a.n)
        qw = RowQWeight.from_f32(w, a.kind)
        x = torch.randn(a.m, a.k, device="cuda")
        bias = torch.zeros(a.n, device="cuda")
        y = torch.empty(a.m, a.n, device="cuda")
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        st = torch.cuda.current_stream().cuda_stream
        for i in range(a.reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            qw.linear_dev(x.data_ptr(), bias.data_ptr(), y.data_ptr(), a.m, C.c_void_p(st))
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            byts = a.k * a.n / (2 if a.kind else 1) + 4 * a.k + 4 * a.m * (a.k + a.n)
            print(f"rowq {'int4' if a.kind else 'int8'} M={a.m} K={a.k} N={a.n}: {ms * 1e3:.1f} us, {byts / ms / 1e6:.1f} GB/s, "
                  f"{2 * a.m * a.k * a.n / ms / 1e9:.2f} TFLOP/s")
        return
    if a.case.startswith("llama"):
        return llama_case(a)
    sm = synth.named(a.model, seed=0, math_mode=a.math)
    V, T = sm.dims[5], sm.dims[4]
    gm = fcb.CudaSlm(sm.config, sm.weights)
    if a.case == "decode":
        prompt = synth.token_ids(0, a.prompt, V)
        gm.set_decode_mode(a.mode)
        for i in range(a.reps):
            t0 = time.perf_counter()
            toks, _ = gm.generate_tokens(prompt, a.tokens)
            print(f"decode {a.tokens} tokens: device {gm.last_decode_ms / a.tokens * 1e3:.1f} us/token, "
                  f"wall {time.perf_counter() - t0:.4f} s, launches {fcb.take_launch_count()}")
        if a.trace and a.mode == 0:
            # phase timeline of one token of the persistent kernel (CTA 0), averaged over blocks
            gm.set_trace(True)
            gm.generate_tokens(prompt, a.tokens)
            t = gm.read_trace()
            gm.set_trace(False)
            L = sm.dims[0]
            names = ["ln1", "qkv", "barrier", "attn", "barrier", "combine", "out", "barrier", "load+ln2", "up",
                     "barrier", "load", "down", "barrier", "load"]
            if len(t) >= 1 + 15 * L:
                body = np.diff(t[:1 + 15 * L])
                per = body.reshape(L, 15)
                print("phase timeline of CTA 0 (ns, mean over blocks):")
                for i, nme in enumerate(names):
                    print(f"  {nme:10s} {per[:, i].mean():9.0f}")
                print(f"  blocks total {body.sum():9.0f} ns; head+select {t[-1] - t[15 * L]:9.0f} ns; token {t[-1]:9.0f} ns")
                print("  head marks:", np.diff(t[15 * L:]).tolist())
    else:
        ids = synth.token_ids(1, a.windows * T, V).reshape(a.windows, T)
        for i in range(a.reps):
            scores, _ = gm.score_sequences(ids, batch_windows=a.windows)
            print(f"score {a.windows} x {T}: device {gm.last_score_ms:.2f} ms, "
                  f"{a.windows * T / gm.last_score_ms * 1e3:.0f} positions/s, launches {fcb.take_launch_count()}")
    gm.close()


def llama_case(a):
    from ferrum_cpu_b200.engine import sampling
    from ferrum_cpu_b200.llama import CudaLlama
    name = a.model if a.model.startswith("llama") else "llama-1b"
    sm = synth.llama_named(name, seed=0, math_mode=a.math)
    c = sm.dims
    gm = CudaLlama.from_synth(sm)
    if a.case == "llama-decode":
        prompt = synth.token_ids(0, a.prompt, c["vocab"])
        cache = gm.new_cache()
        kvd = c["n_kv_head"] * c["head_dim"]
        for i in range(a.reps):
            toks, _ = gm.generate(prompt, a.tokens, sampling(temperature=0.0), cache=cache)
            us = cache.last_decode_ms / a.tokens * 1e3
            # bytes one token streams: Q8_0 matrices once + the f32 KV rows of the mean position
            kv = c["n_layer"] * 2 * (a.prompt + a.tokens / 2) * kvd * 4
            print(f"{name} decode {a.tokens} tokens: device {us:.1f} us/token, {1e6 / us:.0f} tokens/s, "
                  f"{(sm.q8_weight_bytes + kv) / us / 1e3:.0f} GB/s algorithmic, launches {fcb.take_launch_count()}")
    else:
        T = min(c["ctx"], 1024)
        ids = synth.token_ids(1, a.windows * T, c["vocab"]).reshape(a.windows, T)
        qd = c["n_head"] * c["head_dim"]
        flop = 2 * sm.q8_weight_bytes * 32 / 34 + c["n_layer"] * 4 * qd * (T + 1) / 2
        for i in range(a.reps):
            gm.score_sequences(ids, batch_windows=a.windows)
            ms = gm.last_score_ms
            print(f"{name} score {a.windows} x {T}: device {ms:.2f} ms, {a.windows * T / ms * 1e3:.0f} positions/s, "
                  f"{flop * a.windows * T / ms / 1e9:.1f} TFLOP/s algorithmic, launches {fcb.take_launch_count()}")
    gm.close()


if __name__ == "__main__":
    main()
