"""The C-ABI library loads on a machine without a GPU and exports every symbol the public
header declares; device entry points fail with FC_E_CUDA instead of computing on the CPU."""
import os
import re

import numpy as np
import pytest

import ferrum_cpu_b200 as fcb
from ferrum_cpu_b200 import _lib, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ferrum_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fc_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 25
    L = _lib.lib()
    for n in names:
        assert hasattr(L, n), f"{n} is declared in ferrum_cuda.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) <= set(names)


def test_no_cpu_fallback_without_a_device():
    if fcb.device_count() > 0:
        pytest.skip("a B200 is present")
    sm = synth.SynthModel(1, 32, 1, 32, 8, 64, seed=1)
    with pytest.raises(fcb.FerrumCudaError) as e:
        fcb.CudaSlm(sm.config, sm.weights)
    assert e.value.code == _lib.FC_E_CUDA
    with pytest.raises(fcb.FerrumCudaError):
        fcb.q8_0_linear(np.zeros((1, 32), np.float32), synth.q8_0_quantize(np.zeros(64 * 32, np.float32)), None, 64)


def test_argument_validation_precedes_device_use():
    sm = synth.SynthModel(1, 32, 1, 32, 8, 64, seed=1)
    bad = _lib.FcConfig(1, 48, 5, 32, 8, 64, 1, 0)      # 48 % 5 != 0
    with pytest.raises(fcb.FerrumCudaError) as e:
        fcb.CudaSlm(bad, sm.weights)
    assert e.value.code == _lib.FC_E_DIM
    bad = _lib.FcConfig(1, 48, 3, 32, 8, 64, 1, 0)      # 48 % 32 != 0: not Q8_0 eligible
    with pytest.raises(fcb.FerrumCudaError) as e:
        fcb.CudaSlm(bad, sm.weights)
    assert e.value.code == _lib.FC_E_FORMAT


def test_llama_validation_precedes_device_use():
    from ferrum_cpu_b200.llama import CudaLlama
    shape = list(synth.LLAMA_SHAPES["llama-tiny"])
    bad = list(shape)
    bad[3], bad[4], bad[5] = 6, 4, 16                    # 6 query heads cannot share 4 key/value heads (llm.rs:243-247)
    for sm in (synth.SynthLlama(*bad), synth.llama_named("llama-tiny", rope_dim=5), synth.llama_named("llama-tiny", rope_dim=32),
               synth.llama_named("llama-tiny", rope_linear_factor=0.0),
               synth.llama_named("llama-tiny", freq_factors=[1.0, 0.0] * 4)):
        with pytest.raises(fcb.FerrumCudaError) as e:
            CudaLlama.from_synth(sm)
        assert e.value.code == _lib.FC_E_DIM
    if fcb.device_count() == 0:
        with pytest.raises(fcb.FerrumCudaError) as e:
            CudaLlama.from_synth(synth.llama_named("llama-tiny"))
        assert e.value.code == _lib.FC_E_CUDA


def test_rust_binding_declares_every_symbol_of_the_header():
    """ferrum_cuda/src/ffi.rs (the binding a Ferrum maintainer adds; it cannot be compiled here) names every
    function include/ferrum_cuda.h declares, with the same number of arguments."""
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = re.sub(r"/\*.*?\*/", "", open(os.path.join(root, "include", "ferrum_cuda.h")).read(), flags=re.S)
    rust = open(os.path.join(root, "ferrum_cuda", "src", "ffi.rs")).read()
    decls = re.findall(r"\b(fc_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", header)
    assert len(decls) >= 70
    for name, args in decls:
        m = re.search(r"pub fn %s\(([^)]*)\)" % name, rust)
        assert m, f"{name} is missing from ffi.rs"
        n_c = 0 if args.strip() in ("", "void") else args.count(",") + 1
        n_rs = 0 if not m.group(1).strip() else m.group(1).count(",") + 1
        assert n_c == n_rs, f"{name}: {n_c} arguments in the header, {n_rs} in ffi.rs"
