"""Bounded device-side waits: a wait that runs out becomes FC_E_TIMEOUT, the kernel returns, and the
handle keeps working. The failure is made without faulting, trapping or hanging anything: a test hook
(fc_debug_set_wait_budget) shortens the cycle budget of the waits and makes the producer warps of the
pipelined kernels copy nothing, so the consumers' first wait runs out after about a tenth of a
millisecond; every role of the kernel then takes its abort path (stop issuing, give tensor memory back,
wait - with the same limit - for copies in flight) and the launch ends by itself."""
import ctypes as C

import numpy as np
import pytest

import ferrum_cpu_b200 as fcb
from ferrum_cpu_b200 import _lib, synth
from tests import oracle as O

pytestmark = pytest.mark.gpu
SHORT = 200_000          # cycles: about 0.1 ms
DEFAULT = 4_000_000_000


class short_waits_without_producers:
    def __enter__(self):
        _lib.check(_lib.lib().fc_debug_set_wait_budget(SHORT, 1))

    def __exit__(self, *exc):
        _lib.check(_lib.lib().fc_debug_set_wait_budget(DEFAULT, 0))


def test_tensor_core_linear_times_out_and_recovers():
    import torch

    n, k, m = 512, 768, 300
    wq = synth.q8_0_quantize(synth.Rng(5).normal(n * k, 0.02))
    qw = fcb.QWeight(wq, n, k)
    x = torch.from_numpy(synth.Rng(7).normal(m * k, 1.0).reshape(m, k)).cuda()
    y = torch.zeros(m, n, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    with short_waits_without_producers():
        with pytest.raises(fcb.FerrumCudaError) as e:
            qw.linear_dev_noalloc(x.data_ptr(), None, y.data_ptr(), m, stream)     # waits for the stream, reads the status word
        assert e.value.code == _lib.FC_E_TIMEOUT
    torch.cuda.synchronize()                                                        # the kernel has returned; the context is intact
    qw.linear_dev_noalloc(x.data_ptr(), None, y.data_ptr(), m, stream)              # the same handle, a normal call
    ref = x.double() @ torch.from_numpy(synth.q8_0_dequantize(wq, n * k).reshape(n, k)).double().cuda().T
    assert (y.double() - ref).abs().max().item() <= 1e-4 * ref.abs().max().item()
    qw.close()


def test_scoring_times_out_and_recovers():
    sm = synth.named("tiny", seed=0, math_mode=fcb.FC_MATH_BF16X3)
    # head_dim 32: the window forward takes the tensor-core GEMM and the CUDA-core attention
    gm = fcb.CudaSlm(sm.config, sm.weights)
    om = O.OracleModel(sm, threads=2)
    ids = synth.token_ids(1, 128, sm.dims[5])
    with short_waits_without_producers():
        with pytest.raises(fcb.FerrumCudaError) as e:
            gm.token_logprobs(ids, 1)
        assert e.value.code == _lib.FC_E_TIMEOUT
    score, lp, _ = gm.token_logprobs(ids, 1, per_token=True)
    _, _, _, want, _ = om.token_logprobs(ids, 1)
    assert np.abs(lp - want).max() < 1e-3
    gm.close()


def test_persistent_decode_times_out_and_recovers():
    sm = synth.named("tiny", seed=0, perturb=True)
    gm = fcb.CudaSlm(sm.config, sm.weights)
    om = O.OracleModel(sm, threads=2)
    ids = synth.token_ids(3, 6, sm.dims[5])
    for t in ids[:3]:
        gm.feed(t)
        om.feed(t)
    assert gm.cached_len() == 3
    with short_waits_without_producers():
        with pytest.raises(fcb.FerrumCudaError) as e:
            gm.feed(ids[3])                      # one cooperative launch: every CTA's first wait runs out
        assert e.value.code == _lib.FC_E_TIMEOUT
    assert gm.cached_len() == 3                  # the failed step fed nothing
    for t in ids[3:]:                            # the same stream goes on as if nothing had happened
        pg, po = gm.feed(t), om.feed(t)
        assert np.abs(np.log(np.maximum(pg, 1e-12)) - np.log(np.maximum(po, 1e-12))).max() < 2e-4
    assert gm.cached_len() == 6
    gm.close()
