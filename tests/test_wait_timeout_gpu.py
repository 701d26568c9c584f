"""The bounded-wait error path on a GPU, without faulting or hanging it: a kernel whose mbarrier
wait can never be satisfied gives up after a short limit, the host reads the error at the next
synchronisation, and the context keeps working."""
import time

import numpy as np
import pytest

from kandle_b200 import core, lib
from kandle_b200.core import Tensor

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_is_reported_and_the_context_survives(backend):
    backend.synchronize()
    t0 = time.perf_counter()
    lib.call("kd_selftest_wait_timeout", 300)          # 300 us limit; the real kernels use ~1 s
    assert time.perf_counter() - t0 < 5.0
    with pytest.raises(lib.KandleCudaError, match="901"):
        backend.synchronize()
    # the error word was consumed; the same context computes correctly afterwards
    backend.synchronize()
    x = Tensor(np.arange(1024, dtype=np.float32))
    assert np.array_equal(core.add(x, x).dataAsync(), 2 * np.arange(1024, dtype=np.float32))
    # and a second timeout is reported again
    lib.call("kd_selftest_wait_timeout", 50)
    with pytest.raises(lib.KandleCudaError, match="901"):
        backend.synchronize()
    backend.synchronize()


def test_limit_is_validated(backend):
    with pytest.raises(lib.KandleCudaError):
        lib.call("kd_selftest_wait_timeout", 0)
    with pytest.raises(lib.KandleCudaError):
        lib.call("kd_selftest_wait_timeout", 10_000_000)
