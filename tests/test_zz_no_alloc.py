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


def test_noalloc_linear_takes_no_device_memory_after_its_first_call():
    """The claim the entry point exists for: once the first call on a device has made the driver load the
    library's device code (which is when the fixed array comes into being), a call changes the amount of
    free device memory by nothing."""
    import torch

    n, k, m = 512, 768, 200
    qw = fcb.QWeight(synth.q8_0_quantize(synth.Rng(15).normal(n * k, 0.02)), n, k)
    x = torch.from_numpy(synth.Rng(16).normal(m * k, 1.0).reshape(m, k)).cuda()
    y = torch.zeros(m, n, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    qw.linear_dev_noalloc(x.data_ptr(), None, y.data_ptr(), m, stream)      # warm-up: loads the module
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        qw.linear_dev_noalloc(x.data_ptr(), None, y.data_ptr(), m, stream)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    qw.close()


def test_device_pointer_entries_refuse_misaligned_pointers_on_the_host():
    """x_dev / y_dev / bias_dev are accessed with 16-byte vector loads and stores: a pointer off that
    alignment is an FC_E_ARG from the host-side check, and nothing is launched."""
    import torch

    n, k, m = 128, 64, 4
    qw = fcb.QWeight(synth.q8_0_quantize(synth.Rng(17).normal(n * k, 0.02)), n, k)
    x = torch.zeros(m * k + 4, device="cuda")
    y = torch.zeros(m * n + 4, device="cuda")
    for xp, yp in ((x.data_ptr() + 4, y.data_ptr()), (x.data_ptr(), y.data_ptr() + 4)):
        with pytest.raises(fcb.FerrumCudaError) as e:
            qw.linear_dev_noalloc(xp, None, yp, m, None)
        assert e.value.code == _lib.FC_E_ARG
        with pytest.raises(fcb.FerrumCudaError) as e:
            qw.linear_dev(xp, None, yp, m, fcb.FC_MATH_BF16X3, None)
        assert e.value.code == _lib.FC_E_ARG
    fcb.take_launch_count()
    with pytest.raises(fcb.FerrumCudaError):
        qw.linear_dev(x.data_ptr() + 4, None, y.data_ptr(), 1, fcb.FC_MATH_FP32, None)
    assert fcb.take_launch_count() == 0
    qw.close()
