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


def _call(entry, q, kc, vc, ctx, splits, ctx_dev, out):
    lib.call(entry, _r(q), _r(kc), _r(vc), _r(ctx_dev), int(ctx), ctypes.c_float(1.0 / math.sqrt(q.shape[-1])), splits, _r(out))


def _footprint(backend):
    """Everything the library holds on the device: allocator figures plus the scratch buffer it
    obtains from CUDA directly."""
    ws = ctypes.c_uint64(0)
    lib.call("kd_workspace_bytes", ctypes.byref(ws))
    return dict(backend.memory_stats(), workspace=ws.value)


def test_noalloc_decode_attention_matches_the_allocating_entry_point_twice(backend, oracle):
    """Two different problems back to back through the built-in buffer (the second has fewer splits
    and a shorter context, so partials of the first call lie right beside its own), then a call whose
    context length comes from device memory.  The calls of the no-alloc entry point come FIRST and
    alone between two readings of the library's device footprint, which must not move: not the
    allocator's in-use / cached / reserved bytes, and not the scratch buffer kd_attention_decode grows.
    The built-in buffer is filled with NaN patterns before each call: nothing in it needs clearing
    because every slot a call reads is written by that same call.  (All calls here are on the
    library's one stream; two calls overlapping on the GPU would race for the shared buffer.)"""
    b, hq, hkv, max_s, d = 4, 16, 8, 768, 128
    kc = Tensor(synth.normal("na.k", (b, hkv, max_s, d)), dtype="bfloat16")
    vc = Tensor(synth.normal("na.v", (b, hkv, max_s, d)), dtype="bfloat16")
    kc_host, vc_host = kc.dataAsync(), vc.dataAsync()
    problems = [(700, 5, "na.q0", None), (130, 2, "na.q1", None), (0, 0, "na.q2", Tensor(np.array([333], np.int32)))]
    qs = [lib.round_to_bf16(synth.normal(seed, (b, hq, 1, d))) for _, _, seed, _ in problems]
    tq = [Tensor(q, dtype="bfloat16") for q in qs]
    outs = [Tensor(np.full((b, hq, 1, d), np.nan, np.float32), dtype="bfloat16") for _ in problems]
    lib.call("kd_debug_fill_scratch", 0xFF)
    backend.synchronize()
    before = _footprint(backend)
    for (ctx, splits, _, ctx_dev), q, out in zip(problems, tq, outs):
        lib.call("kd_debug_fill_scratch", 0xFF)          # a memset on the stream, no allocation
        _call("kd_attention_decode_noalloc", q, kc, vc, ctx, splits, ctx_dev, out)
    backend.synchronize()
    assert _footprint(backend) == before, "kd_attention_decode_noalloc changed the library's device footprint"
    for call, ((ctx, splits, _, ctx_dev), qh, q, out) in enumerate(zip(problems, qs, tq, outs)):
        got = out.dataAsync()
        want_t = core.empty(q.shape, "bfloat16")
        _call("kd_attention_decode", q, kc, vc, ctx, splits, ctx_dev, want_t)
        want = want_t.dataAsync()
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max(), f"call {call}: differs from kd_attention_decode"
        n = ctx if ctx_dev is None else 333
        ref = oracle.sdpa(qh, kc_host[:, :, :n], vc_host[:, :, :n], is_causal=False)
        assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max(), f"call {call}: differs from the oracle"


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
