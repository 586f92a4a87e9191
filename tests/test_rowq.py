"""Per-row-scale int8 / int4 weights (quant.rs:122-263) and their linear (ops.rs:268-377): the
oracle restatement pinned on the reference's unit tests (CPU), the library's host codec against
it (CPU), and the CUDA kernel against the oracle (GPU)."""
import numpy as np
import pytest

import ferrum_cpu_b200 as fcb
from ferrum_cpu_b200 import _lib, engine
from tests import oracle as O
from tests.test_llama_oracle import det

INT8, INT4 = _lib.FC_Q_INT8, _lib.FC_Q_INT4


def f32_linear(x, w, bias):
    return O.linear(x, np.ascontiguousarray(w, dtype=np.float32), bias, threads=2)


# ---- quant.rs:597-685 -------------------------------------------------------------------
def test_int8_roundtrip_bounded_by_half_scale():
    rows, cols = 5, 40
    data = (np.sin(np.arange(rows * cols, dtype=np.float32) * np.float32(0.017)) * np.float32(1.3)).astype(np.float32).reshape(rows, cols)
    q, scales = O.rowq_from_f32(data, INT8)
    assert q.size + scales.size * 4 == rows * cols + rows * 4          # resident_bytes
    back = O.rowq_to_f32(q, scales, rows, cols, INT8)
    for r in range(rows):
        scale = np.abs(data[r]).max() / np.float32(127.0)
        assert scales[r] == np.float32(scale)
        assert np.abs(data[r] - back[r]).max() <= scale * 0.5 + 1e-6


def test_int4_roundtrip_bounded_by_half_step_with_odd_width():
    rows, cols = 4, 31
    data = np.cos(np.arange(rows * cols, dtype=np.float32) * np.float32(0.07)).astype(np.float32).reshape(rows, cols)
    q, scales = O.rowq_from_f32(data, INT4)
    assert q.size == rows * 16                                          # ceil(31 / 2) bytes per row
    back = O.rowq_to_f32(q, scales, rows, cols, INT4)
    for r in range(rows):
        step = np.abs(data[r]).max() / np.float32(7.0)
        assert np.abs(data[r] - back[r]).max() <= step * 0.5 + 1e-6


def test_packed_sizes_and_nibbles():
    L = O.lib()
    assert L.fo_rowq_packed_len(64, 64, INT4) == 64 * 64 // 2 and L.fo_rowq_packed_len(64, 64, INT8) == 64 * 64
    assert L.fo_rowq_packed_len(3, 5, INT8) == 3 * 5 and L.fo_rowq_packed_len(3, 5, INT4) == 3 * 3
    assert [L.fo_nibble_to_i8(n) for n in (0x0, 0x7, 0xF, 0x9)] == [0, 7, -1, -7]
    q, scales = O.rowq_from_f32(np.zeros((2, 8), np.float32), INT8)     # an all-zero row: scale 0, levels 0
    assert not q.any() and not scales.any()


# ---- ops.rs:836-949 ---------------------------------------------------------------------
def test_qlinear_int8_close_to_f32_linear_and_int4_tracks_it():
    k, n = 96, 200
    for seed, kind, check in ((7, INT8, lambda d: d.max() < 0.05), (11, INT4, lambda d: d.mean() < 0.5)):
        w = det(k * n, seed).reshape(k, n)
        bias, x = det(n, seed + 1), det(k, seed + 2).reshape(1, k)
        q, scales = O.rowq_from_f32(w, kind)
        got = O.rowq_linear(x, q, scales, kind, bias, n)
        assert check(np.abs(got - f32_linear(x, w, bias)))


def test_qlinear_equals_the_dequantised_serial_sum():
    for (m, k, n, kind) in ((1, 64, 2048, INT8), (1, 8, 8, INT8), (4, 64, 300, INT8), (4, 64, 300, INT4), (2, 33, 31, INT4)):
        w = det(k * n, 21).reshape(k, n)
        bias, x = det(n, 22), det(m * k, 23).reshape(m, k)
        q, scales = O.rowq_from_f32(w, kind)
        wf = O.rowq_to_f32(q, scales, k, n, kind)
        want = bias[None, :].astype(np.float64) + x.astype(np.float64) @ wf.astype(np.float64)
        assert np.abs(O.rowq_linear(x, q, scales, kind, bias, n) - want).max() < 1e-3


# ---- the library's host codec against the oracle ------------------------------------------
@pytest.mark.parametrize("kind", [INT8, INT4])
@pytest.mark.parametrize("shape", [(5, 40), (4, 31), (64, 64), (3, 5), (7, 1)])
def test_host_codec_is_bit_identical_to_the_oracle(kind, shape):
    rows, cols = shape
    data = (det(rows * cols, 5) * np.float32(1.7)).reshape(rows, cols)
    data[0, 0] = 0.0
    q, scales = engine.rowq_from_f32(data, kind)
    oq, oscales = O.rowq_from_f32(data, kind)
    assert np.array_equal(q, oq) and np.array_equal(scales, oscales)
    assert np.array_equal(engine.rowq_to_f32(q, scales, rows, cols, kind), O.rowq_to_f32(oq, oscales, rows, cols, kind))


# ---- the CUDA kernel -----------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("kind", [INT8, INT4])
@pytest.mark.parametrize("m,k,n", [(1, 64, 2048), (1, 2048, 2048), (1, 2048, 8192), (1, 96, 200), (1, 8, 8), (2, 33, 31),
                                   (4, 64, 300), (8, 512, 1000), (9, 256, 517), (64, 1024, 1024)])
def test_rowq_linear_matches_oracle(kind, m, k, n):
    w = (det(k * n, 31) * np.float32(0.05)).reshape(k, n)
    bias, x = det(n, 32), det(m * k, 33).reshape(m, k)
    q, scales = engine.rowq_from_f32(w, kind)
    want = O.rowq_linear(x, q, scales, kind, bias, n)
    qw = engine.RowQWeight(q, scales, k, n, kind)
    got = qw.linear(x, bias)
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max() + 1e-5
    assert np.array_equal(got, qw.linear(x, bias))                      # fixed reduction order: bitwise repeatable
    qw.close()


@pytest.mark.gpu
def test_rowq_linear_rejects_bad_shapes():
    qw = engine.RowQWeight.from_f32(det(3 * 4, 1).reshape(3, 4), INT8)
    with pytest.raises(fcb.FerrumCudaError) as e:
        qw.linear(np.zeros((1, 5), np.float32), np.zeros(4, np.float32))   # ops.rs:952-957
    assert e.value.code == _lib.FC_E_DIM
    with pytest.raises(fcb.FerrumCudaError) as e:
        qw.linear(np.zeros((1, 3), np.float32), np.zeros(2, np.float32))   # ops.rs:958-960
    assert e.value.code == _lib.FC_E_DIM
