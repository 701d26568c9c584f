"""Key `randn` on the GPU against the CPU restatement of the reference's Philox4x32-10 + Box-Muller
kernel.  The integer part (counters, keys, Philox words) is exact; the float part goes through
log / sqrt / cos of two different math libraries, so values are compared at 2e-6 of the largest
|z| the stream produces (about 5.5), bf16 outputs at one bf16 rounding."""
import ctypes

import numpy as np
import pytest

from kandle_b200 import core, lib
from kandle_b200.core import Tensor

pytestmark = pytest.mark.gpu


def _randn(t, seed, base=0, mean=0.0, std=1.0, row0=0, col0=0, full_cols=0):
    lib.call("kd_randn", ctypes.byref(t._handle.c()), ctypes.c_uint64(seed), ctypes.c_uint32(base), ctypes.c_float(mean),
             ctypes.c_float(std), row0, col0, full_cols)
    return t.dataAsync()


def test_randn_matches_the_oracle_stream(backend, oracle):
    n = 1 << 20
    got = _randn(core.empty((n + 1,), "float32"), 0x1234567890ABCDEF, base=4294967290)   # counter wraps mod 2^32
    ref = oracle.randn(n + 1, 0x1234567890ABCDEF, 4294967290)
    assert np.abs(got - ref).max() <= 2e-6 * 5.5
    got = _randn(core.empty((257, 33), "float32"), 7, mean=0.5, std=0.02)
    ref = np.float32(0.5) + np.float32(0.02) * oracle.randn(257 * 33, 7).reshape(257, 33)
    assert np.abs(got - ref).max() <= 1e-6


def test_randn_slices_hold_what_the_full_matrix_holds(backend, oracle):
    rows, cols = 96, 200
    full = _randn(core.empty((rows, cols), "bfloat16"), 99, std=0.02)
    ref = lib.round_to_bf16(np.float32(0.02) * oracle.randn(rows * cols, 99).reshape(rows, cols))
    assert np.abs(full - ref).max() <= 0.02 * 5.5 * 2.0 ** -8         # one bf16 rounding of values that differ by 1e-7
    assert (full != ref).mean() < 1e-3
    # row slice (column-parallel weight) and column slice (row-parallel weight), odd offsets included
    part = _randn(core.empty((24, cols), "bfloat16"), 99, std=0.02, row0=48, col0=0, full_cols=cols)
    assert np.array_equal(part, full[48:72])
    part = _randn(core.empty((rows, 37), "bfloat16"), 99, std=0.02, row0=0, col0=101, full_cols=cols)
    assert np.array_equal(part, full[:, 101:138])
    # into a strided destination: rows 3.. of a wider buffer
    wide = core.zeros((rows + 3, cols), "bfloat16")
    view = wide.slice([slice(3, None), slice(0, 64)])
    _randn(view, 99, std=0.02, row0=0, col0=64, full_cols=cols)
    w = wide.dataAsync()
    assert np.array_equal(w[3:, :64], full[:, 64:128]) and not w[:3].any() and not w[:, 64:].any()


def test_randn_key_consumes_the_generator_offset(backend, oracle):
    core.manualSeed(42)
    a = core.randn((5, 7)).dataAsync()
    b = core.randn((6,)).dataAsync()
    ref_a = oracle.randn(35, 42, 0).reshape(5, 7)
    ref_b = oracle.randn(6, 42, 18)              # 35 numbers consumed ceil(35 / 2) = 18 Philox calls
    assert np.abs(a - ref_a).max() <= 2e-5 and np.abs(b - ref_b).max() <= 2e-5
    core.manualSeed(42)
    assert np.array_equal(core.randn((5, 7)).dataAsync(), a)


def test_randn_rejects_bad_slices(backend):
    t = core.empty((4, 8), "float32")
    with pytest.raises(lib.KandleCudaError):
        _randn(t, 1, col0=4, full_cols=10)       # columns 4..12 of a 10-column matrix
    with pytest.raises(lib.KandleCudaError):
        _randn(core.empty((4,), "int32"), 1)
