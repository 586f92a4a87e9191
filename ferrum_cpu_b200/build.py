"""Builds libferrum_cuda.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m ferrum_cpu_b200.build [--verbose]
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libferrum_cuda.so")
SOURCES = ["codec.cpp", "gguf_load.cpp", "gemv.cu", "gemv_stream.cu", "rowops.cu", "attn.cu", "gemm_simt.cu", "gemm_tc.cu", "attn_tc.cu", "decode_mega.cu", "decode_batch.cu", "sample.cu", "llama_ops.cu", "llama.cu", "rowq.cu", "ggml_linear.cu", "api.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
]


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _compile(src, verbose):
    obj = os.path.join(OBJ, src + ".o")
    deps = [os.path.join(CSRC, src)] + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    deps.append(os.path.join(HERE, "..", "include", "ferrum_cuda.h"))
    if _newer(obj, deps):
        return obj, ""
    cmd = ["nvcc", *NVCC_FLAGS, "-x", "cu", "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose), SOURCES))
    objs = [o for o, _ in results]
    log = "".join(l for _, l in results)
    if not _newer(LIB, objs):
        cmd = ["nvcc", "-shared", "-o", LIB, *objs, "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return log


if __name__ == "__main__":
    out = build(verbose="--verbose" in sys.argv)
    if out:
        print(out)
    print(LIB)
