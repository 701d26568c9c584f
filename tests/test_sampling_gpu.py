"""GPU parity of kd_sample (temperature / top-k / top-p / draw / greedy) against the oracle's
restatement of the reference's host-side sampler (packages/model-utils/src/sampling/index.ts:103-238).
The same row of logits is drawn with many uniform numbers so that the cumulative-sum boundaries are
exercised; token ids must agree exactly."""
import ctypes

import numpy as np
import pytest

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor

pytestmark = pytest.mark.gpu


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


def _run(logits, temperature, top_k, top_p, do_sample, uniforms):
    B = logits.shape[0]
    lt = Tensor(logits)
    ut = Tensor(np.asarray(uniforms, dtype=np.float32)) if do_sample else None
    ids = core.zeros((B,), "int64")
    lp = core.zeros((B,), "float32")
    lib.call("kd_sample", _r(lt), ctypes.c_double(temperature), int(top_k), ctypes.c_double(top_p), int(do_sample), _r(ut),
             _r(ids), _r(lp))
    return ids.dataAsync(), lp.dataAsync()


CONFIGS = [
    (1.0, 0, 1.0), (0.7, 50, 1.0), (1.0, 0, 0.9), (0.8, 40, 0.95), (1.3, 5, 0.5), (0.5, 1, 1.0), (2.0, 1000, 0.999),
    (1.0, 3, 0.01),
]


@pytest.mark.parametrize("temperature,top_k,top_p", CONFIGS)
@pytest.mark.parametrize("V", [151936, 1000])
def test_sampling_matches_the_oracle_for_many_uniforms(backend, oracle, temperature, top_k, top_p, V):
    n = 48
    row = synth.normal(f"sample-logits-{V}", (V,), 2.5)
    us = (np.arange(n, dtype=np.float64) + 0.37) / n
    us = np.concatenate([us, [0.0, 0.999999]]).astype(np.float32)
    logits = np.tile(row, (us.size, 1))
    ids, lp = _run(logits, temperature, top_k, top_p, True, us)
    for j, u in enumerate(us):
        ref = oracle.sample(row, temperature, top_k, top_p, True, float(u))
        assert ids[j] == ref["token"], f"u={u}: got {ids[j]}, oracle {ref['token']}"
        assert abs(lp[j] - ref["logprob"]) <= 1e-5 * max(1.0, abs(ref["logprob"]))


def test_ties_follow_the_stable_sort(backend, oracle):
    """Quantised logits: the top-k / top-p cut falls inside a group of equal values, of which the
    reference's stable sort keeps the lowest indices."""
    V = 4096
    row = np.round(synth.normal("sample-ties", (V,), 1.5) * 2.0) / 2.0
    row[[7, 99, 1234]] = 0.0
    row[55] = -0.0
    us = ((np.arange(64) + 0.5) / 64).astype(np.float32)
    logits = np.tile(row.astype(np.float32), (us.size, 1))
    for temperature, top_k, top_p in [(1.0, 10, 1.0), (1.0, 37, 1.0), (0.9, 0, 0.3), (1.1, 200, 0.6), (1.0, 500, 0.97)]:
        ids, lp = _run(logits, temperature, top_k, top_p, True, us)
        for j, u in enumerate(us):
            ref = oracle.sample(row, temperature, top_k, top_p, True, float(u))
            assert ids[j] == ref["token"], f"cfg {(temperature, top_k, top_p)} u={u}: got {ids[j]}, oracle {ref['token']}"
            assert abs(lp[j] - ref["logprob"]) <= 1e-5 * max(1.0, abs(ref["logprob"]))


def test_greedy_and_small_vocabularies(backend, oracle):
    for V in (1, 5, 33, 1025):
        logits = synth.normal(f"sample-small-{V}", (6, V), 3.0)
        logits[0, :] = 1.25                      # every value equal: index 0 wins
        ids, lp = _run(logits, 0.7, 0, 1.0, False, None)
        for b in range(6):
            ref = oracle.sample(logits[b], 0.7, 0, 1.0, False)
            assert ids[b] == ref["token"]
            assert abs(lp[b] - ref["logprob"]) <= 1e-5 * max(1.0, abs(ref["logprob"]))
        us = np.linspace(0.01, 0.99, 6).astype(np.float32)
        ids, lp = _run(logits, 1.2, 3, 0.8, True, us)
        for b in range(6):
            ref = oracle.sample(logits[b], 1.2, 3, 0.8, True, float(us[b]))
            assert ids[b] == ref["token"]


def test_argument_checks(backend):
    lt = Tensor(np.zeros((2, 16), np.float32))
    ids = core.zeros((2,), "int64")
    u = Tensor(np.zeros((2,), np.float32))
    with pytest.raises(lib.KandleCudaError):     # temperature must be positive
        lib.call("kd_sample", _r(lt), ctypes.c_double(0.0), 0, ctypes.c_double(1.0), 1, _r(u), _r(ids), None)
    with pytest.raises(lib.KandleCudaError):     # sampling needs uniforms
        lib.call("kd_sample", _r(lt), ctypes.c_double(1.0), 0, ctypes.c_double(1.0), 1, None, _r(ids), None)
    with pytest.raises(lib.KandleCudaError):     # ids must be int64 [B]
        lib.call("kd_sample", _r(lt), ctypes.c_double(1.0), 0, ctypes.c_double(1.0), 0, None, _r(u), None)
