"""The one-shot peer-memory all-reduce fused with residual add + RMSNorm (kd_allreduce_add_rmsnorm),
on ONE GPU: the ranks are emulated inside one cooperative launch (kd_p2p_emulate), which exercises
the whole protocol (slots, per-row flags, rank-order sum, the call counter) except the NVLink hop.
The multi-GPU form runs in tests/tp_worker.py.  A rank whose flags never arrive is simulated on the
host side of the call (drop_rank): the others' bounded waits run out and the call reports an error
status; nothing hangs and the context stays usable."""
import ctypes

import numpy as np
import pytest

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor

pytestmark = pytest.mark.gpu


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


@pytest.fixture()
def emulated_ranks(backend):
    lib.call("kd_p2p_emulate", 4)
    yield 4
    lib.call("kd_p2p_disconnect")


def _reference(x, resid, w, eps):
    total = x.astype(np.float64).sum(axis=(0, 1)) + resid
    norm = total / np.sqrt((total ** 2).mean(-1, keepdims=True) + eps) * w
    return total, norm


def test_emulated_ranks_sum_in_rank_order_and_normalise(emulated_ranks, backend):
    ranks, splits, rows, n, eps = emulated_ranks, 3, 8, 2560, 1e-6
    w = lib.round_to_bf16(1.0 + synth.normal("p2p.w", (n,), 0.1))
    tw = Tensor(w, dtype="bfloat16")
    resid = synth.normal("p2p.r", (rows, n))
    tr = Tensor(resid)
    for call in range(5):                       # both slots, several tags
        x = synth.normal(f"p2p.x{call}", (ranks, splits, rows, n))
        tx = Tensor(x)
        sums, norms = core.empty((ranks, rows, n), "float32"), core.empty((ranks, rows, n), "bfloat16")
        lib.call("kd_allreduce_add_rmsnorm", _r(tx), _r(tr), _r(tw), ctypes.c_float(eps), _r(sums), _r(norms))
        s, nm = sums.dataAsync(), norms.dataAsync()
        total, norm = _reference(x, resid, w, eps)
        assert np.abs(s[0] - total).max() <= 1e-5 * np.abs(total).max(), f"call {call}"
        assert np.abs(nm[0] - norm).max() <= 2.0 ** -7 * np.abs(norm).max(), f"call {call}"
        for r in range(1, ranks):               # every rank holds the same bits
            assert np.array_equal(s[r], s[0]) and np.array_equal(nm[r], nm[0]), f"call {call}, rank {r}"


def test_a_rank_that_never_publishes_ends_the_call_with_an_error_status(emulated_ranks, backend):
    ranks, rows, n = emulated_ranks, 4, 512
    x = Tensor(synth.normal("p2p.xd", (ranks, 1, rows, n)))
    w = Tensor(np.ones((n,), np.float32), dtype="bfloat16")
    out = core.empty((ranks, rows, n), "bfloat16")
    # rank 2 stays silent; the waits of the others give up after 2e6 clock cycles (about a millisecond)
    lib.call("kd_p2p_selftest_dropped_flag", _r(x), _r(w), _r(out), 2, ctypes.c_uint32(2_000_000))
    with pytest.raises(lib.KandleCudaError) as e:
        backend.synchronize()
    assert e.value.status == 6 and "601" in str(e.value)
    # the next call works: new tag, the other slot
    sums, norms = core.empty((ranks, rows, n), "float32"), core.empty((ranks, rows, n), "bfloat16")
    lib.call("kd_allreduce_add_rmsnorm", _r(x), None, _r(w), ctypes.c_float(1e-6), _r(sums), _r(norms))
    total = x.dataAsync().astype(np.float64).sum(axis=(0, 1))
    assert np.abs(sums.dataAsync()[3] - total).max() <= 1e-5 * np.abs(total).max()


def test_one_shot_all_reduce_refuses_what_it_cannot_hold(emulated_ranks, backend):
    ranks = emulated_ranks
    w = Tensor(np.ones((8192,), np.float32), dtype="bfloat16")
    x = core.empty((ranks, 1, 32, 8192), "float32")            # 32 x 8192 x 4 bytes = 1 MiB fits; 128 rows would not
    out = core.empty((ranks, 32, 8192), "bfloat16")
    lib.call("kd_allreduce_add_rmsnorm", _r(x), None, _r(w), ctypes.c_float(1e-6), None, _r(out))
    backend.synchronize()
    with pytest.raises(lib.KandleCudaError):
        xw = core.empty((ranks, 1, 40, 8192), "float32")       # 160 CTAs exceed one co-resident wave of 148
        ow = core.empty((ranks, 40, 8192), "bfloat16")
        lib.call("kd_allreduce_add_rmsnorm", _r(xw), None, _r(w), ctypes.c_float(1e-6), None, _r(ow))
    with pytest.raises(lib.KandleCudaError):                   # row width not a multiple of 8
        lib.call("kd_allreduce_add_rmsnorm", _r(core.empty((ranks, 1, 2, 12), "float32")), None,
                 _r(Tensor(np.ones((12,), np.float32), dtype="bfloat16")), ctypes.c_float(1e-6), None, _r(core.empty((ranks, 2, 12), "bfloat16")))
