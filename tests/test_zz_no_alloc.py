"""The allocation-free linear (fc_q8_0_linear_dev_noalloc) against the allocating entry point.

Some hosts of this library cannot call cudaMalloc while they serve: all free device memory was
given to their own pool at start-up, or the calling thread must not block on the driver's
allocation lock. For them the library keeps the scratch of the tensor-core linear (the bf16
planes of the activations and a status word) in a fixed device array. This file checks, through
the C ABI, that the variant computes exactly what fc_q8_0_linear_dev computes, twice in a row
(the array keeps the previous call's contents), and that it refuses sizes beyond the array.

Collected last on purpose: a run that stops at the first failure has then already run every
other test."""
import ctypes as C

import numpy as np
import pytest

import ferrum_cpu_b200 as fcb
from ferrum_cpu_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def test_noalloc_linear_matches_the_allocating_entry_point_twice():
    import torch

    n, k = 1000, 768                     # N not a multiple of the 128-row tile
    wq = synth.q8_0_quantize(synth.Rng(5).normal(n * k, 0.02))
    qw = fcb.QWeight(wq, n, k)
    bias = torch.from_numpy(synth.Rng(6).normal(n, 0.5)).cuda()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two calls in a row with different shapes: the second finds the first one's planes and
    # status word in the shared array and must not be affected by them
    for call, m in enumerate((300, 77)):
        x = torch.from_numpy(synth.Rng(7 + call).normal(m * k, 1.0).reshape(m, k)).cuda()
        want = torch.zeros(m, n, device="cuda")
        got = torch.full((m, n), float("nan"), device="cuda")
        qw.linear_dev(x.data_ptr(), bias.data_ptr(), want.data_ptr(), m, fcb.FC_MATH_BF16X3, stream)
        qw.linear_dev_noalloc(x.data_ptr(), bias.data_ptr(), got.data_ptr(), m, stream)
        torch.cuda.synchronize()
        # same kernels on the same inputs: the results are bit-identical, which is inside the
        # 1e-4 relative tolerance the tensor-core tests use
        assert torch.equal(got, want), f"call {call}: max abs diff {(got - want).abs().max().item():.3e}"
        ref = x.double() @ torch.from_numpy(synth.q8_0_dequantize(wq, n * k).reshape(n, k)).double().cuda().T + bias.double()
        assert (got.double() - ref).abs().max().item() <= 1e-4 * ref.abs().max().item()
    qw.close()


def test_noalloc_linear_rejects_sizes_beyond_its_array():
    import torch

    n, k = 128, 4096
    qw = fcb.QWeight(synth.q8_0_quantize(np.zeros(n * k, dtype=np.float32)), n, k)
    m = 1025                              # 1025 * 4096 > 4 Mi activations
    x = torch.zeros(m, k, device="cuda")
    y = torch.zeros(m, n, device="cuda")
    with pytest.raises(fcb.FerrumCudaError) as e:
        qw.linear_dev_noalloc(x.data_ptr(), None, y.data_ptr(), m, None)
    assert e.value.code == _lib.FC_E_SHAPE and "exceeds" in str(e.value)
    qw.linear_dev_noalloc(x.data_ptr(), None, y.data_ptr(), 1024, None)   # exactly at the limit
    torch.cuda.synchronize()
    assert float(y.abs().max()) == 0.0
    qw.close()
