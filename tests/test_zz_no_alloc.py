"""The decode-attention entry point for callers that may not allocate device memory
(kd_attention_decode_noalloc): a serving loop whose memory pool already owns the GPU, or a latency
path that cannot afford a cudaMalloc.  It must give what kd_attention_decode gives, on repeated
calls that reuse the same built-in scratch buffer, and must refuse problems that do not fit it.

Collected last on purpose: a failure here cannot hide the result of any other test in a run that
stops at the first failure."""
import ctypes
import math

import numpy as np
import pytest

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor

pytestmark = pytest.mark.gpu


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


def _run(entry, q, kc, vc, ctx, splits, ctx_dev=None):
    out = core.empty(q.shape, "bfloat16")
    lib.call(entry, _r(q), _r(kc), _r(vc), _r(ctx_dev), int(ctx), ctypes.c_float(1.0 / math.sqrt(q.shape[-1])), splits, _r(out))
    return out.dataAsync()


def test_noalloc_decode_attention_matches_the_allocating_entry_point_twice(backend, oracle):
    b, hq, hkv, max_s, d = 4, 16, 8, 768, 128
    kc = Tensor(synth.normal("na.k", (b, hkv, max_s, d)), dtype="bfloat16")
    vc = Tensor(synth.normal("na.v", (b, hkv, max_s, d)), dtype="bfloat16")
    before = backend.memory_stats()
    # two different problems back to back through the same built-in buffer; the second has fewer
    # splits and a shorter context, so stale partials of the first call sit right next to its own
    for call, (ctx, splits, seed) in enumerate([(700, 5, "na.q0"), (130, 2, "na.q1")]):
        qh = lib.round_to_bf16(synth.normal(seed, (b, hq, 1, d)))
        q = Tensor(qh, dtype="bfloat16")
        want = _run("kd_attention_decode", q, kc, vc, ctx, splits)
        got = _run("kd_attention_decode_noalloc", q, kc, vc, ctx, splits)
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max(), f"call {call}: differs from kd_attention_decode"
        ref = oracle.sdpa(qh, kc.dataAsync()[:, :, :ctx], vc.dataAsync()[:, :, :ctx], is_causal=False)
        assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max(), f"call {call}: differs from the oracle"
    # the context length may also come from device memory
    ctx_dev = Tensor(np.array([333], np.int32))
    q = Tensor(lib.round_to_bf16(synth.normal("na.q2", (b, hq, 1, d))), dtype="bfloat16")
    want = _run("kd_attention_decode", q, kc, vc, 0, 0, ctx_dev)
    got = _run("kd_attention_decode_noalloc", q, kc, vc, 0, 0, ctx_dev)
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
    after = backend.memory_stats()
    assert after["reserved"] >= before["reserved"]          # bookkeeping still consistent


def test_noalloc_decode_attention_refuses_what_does_not_fit(backend):
    # 64 sequences x 32 kv heads x 32 splits x group 4 x 130 floats = 136 MB of partials: beyond the 8 MiB buffer
    b, hq, hkv, max_s, d = 64, 128, 32, 4096, 128
    q = core.empty((b, hq, 1, d), "bfloat16")
    kc = core.empty((b, hkv, max_s, d), "bfloat16")
    out = core.empty((b, hq, 1, d), "bfloat16")
    with pytest.raises(lib.KandleCudaError) as e:
        lib.call("kd_attention_decode_noalloc", _r(q), _r(kc), _r(kc), None, 4096, ctypes.c_float(0.1), 32, _r(out))
    assert e.value.status == 1 and "scratch" in str(e.value) and "8388608" in str(e.value)
    for t in (q, kc, out):
        t.dispose()
