"""Linear layers on weights kept in their GGML block format (fc_ggml_linear): the blocks are decoded inside the kernel.
One-hot activation rows read single weights back, so the in-kernel decoders are held to the numpy restatement of the
reference's decoders (oracle/gguf_dequant.py) value for value; random activations against an f64 product of the decoded
weights."""
import ctypes as C

import numpy as np
import pytest

from ferrum_cpu_b200 import _lib
from tests.test_ggml_formats import GD, random_any

pytestmark = pytest.mark.gpu


class Weight:
    def __init__(self, t, raw, n, k):
        self.h = C.c_void_p()
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        rc = _lib.lib().fc_ggml_weight_upload(0, t, raw.ctypes.data_as(C.c_void_p), raw.size, n, k, C.byref(self.h))
        assert rc == _lib.FC_OK, _lib.lib().fc_last_error()
        self.n, self.k = n, k

    def linear(self, x, bias=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty((x.shape[0], self.n), dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32).ctypes.data_as(C.c_void_p)
        rc = _lib.lib().fc_ggml_linear(self.h, x.ctypes.data_as(C.c_void_p), b, y.ctypes.data_as(C.c_void_p), x.shape[0])
        assert rc == _lib.FC_OK, _lib.lib().fc_last_error()
        return y

    def close(self):
        _lib.lib().fc_ggml_weight_free(self.h)


@pytest.mark.parametrize("t", sorted(GD.BLOCK))
def test_in_kernel_decoders_equal_the_oracle(t):
    n, k = 5, 512
    raw = random_any(t, n * k, 90 + t)
    want = GD.dequantize(t, raw, n * k).reshape(n, k)
    w = Weight(t, raw, n, k)
    # rows of the identity: y[m][:] = W[:, m] exactly (one product by 1.0, the rest zeros)
    got = np.concatenate([w.linear(np.eye(k, dtype=np.float32)[m0:m0 + 64]) for m0 in range(0, k, 64)])   # [k][n]
    assert np.array_equal(got.T, want)        # value for value (a weight of -0.0 comes back as +0.0 through the sum)
    w.close()


@pytest.mark.parametrize("t,m", [(GD.Q4_0, 1), (GD.Q5_0, 3), (GD.Q4_K, 1), (GD.Q6_K, 9), (GD.Q5_K, 2), (GD.Q8_0, 17), (GD.Q2_K, 1), (GD.Q3_K, 4)])
def test_linear_on_block_formats(t, m):
    n, k = 130, 768
    rng = np.random.default_rng(t * 10 + m)
    raw = random_any(t, n * k, 200 + t)
    wf = GD.dequantize(t, raw, n * k).reshape(n, k).astype(np.float64)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    w = Weight(t, raw, n, k)
    want = x.astype(np.float64) @ wf.T + bias
    got = w.linear(x, bias)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 2e-5 * scale + 1e-6
    assert np.abs(w.linear(x) + bias - want).max() <= 2e-5 * scale + 1e-5     # bias may be NULL
    w.close()


def test_refusals():
    L = _lib.lib()
    h = C.c_void_p()
    raw = np.zeros(144 * 4, dtype=np.uint8)
    args = raw.ctypes.data_as(C.c_void_p)
    assert L.fc_ggml_weight_upload(0, 15, args, raw.size, 1, 256, C.byref(h)) == _lib.FC_E_FORMAT      # unknown type
    assert L.fc_ggml_weight_upload(0, GD.Q4_K, args, raw.size, 1, 320, C.byref(h)) == _lib.FC_E_FORMAT  # not whole super-blocks
    assert L.fc_ggml_weight_upload(0, GD.Q4_K, args, raw.size, 8, 256, C.byref(h)) == _lib.FC_E_FORMAT  # data too short
    assert L.fc_ggml_weight_upload(0, GD.Q4_K, args, raw.size, 4, 256, C.byref(h)) == _lib.FC_OK
    L.fc_ggml_weight_free(h)
