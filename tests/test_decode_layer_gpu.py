"""GPU parity of kd_decode_layer_fused (o_proj + residual, gate/up SiLU*up, down + residual, the
next layer's QKV with q/k RMSNorm, rotary embedding and the KV-cache write: one persistent kernel,
four dependent phases, no split-K) against the oracle's unfused operator sequence, i.e. what
packages/model-utils/src/qwen3/decoder_layer.ts:191-241 and attention/gqa.ts:246-322 compute for one
new token per sequence."""
import ctypes

import numpy as np
import pytest

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor
from kandle_b200.engine import interleave_gate_up

pytestmark = pytest.mark.gpu
D = 128


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


def _rb(a):
    return lib.round_to_bf16(np.ascontiguousarray(a, dtype=np.float32))


def _case(mb, H, Ko, I, hq, hkv, seed, max_s=40, pos=17):
    n = lambda name, shape, std=1.0: synth.normal(f"dl.{name}{seed}", shape, std)  # noqa: E731
    c = {
        "attn": _rb(n("attn", (mb, Ko))), "wo": _rb(n("wo", (H, Ko), 0.03)), "h": n("h", (mb, H)),
        "post": _rb(1.0 + n("post", (H,), 0.1)), "wg": _rb(n("wg", (I, H), 0.03)), "wu": _rb(n("wu", (I, H), 0.03)),
        "wd": _rb(n("wd", (H, I), 0.03)), "next": _rb(1.0 + n("next", (H,), 0.1)),
        "hq": hq, "hkv": hkv, "max_s": max_s, "pos": pos,
    }
    if hq:
        c["wq"] = _rb(n("wq", ((hq + 2 * hkv) * D, H), 0.03))
        c["qw"], c["kw"] = _rb(1.0 + n("qw", (D,), 0.1)), _rb(1.0 + n("kw", (D,), 0.1))
    return c


def _oracle(oracle, c, eps):
    """h1, act, h2 and then either x_final or (q, k, v) rows of the new token."""
    h1 = c["h"] + oracle.linear(c["attn"], c["wo"])
    x = _rb(oracle.rms_norm(h1, c["post"], eps))
    act = _rb(oracle.unary("silu", oracle.linear(x, c["wg"])) * oracle.linear(x, c["wu"]))
    h2 = h1 + oracle.linear(act, c["wd"])
    x2 = _rb(oracle.rms_norm(h2, c["next"], eps))
    if not c["hq"]:
        return h1, act, h2, x2, None
    mb, hq, hkv = c["attn"].shape[0], c["hq"], c["hkv"]
    qkv = oracle.linear(x2, c["wq"]).reshape(mb, hq + 2 * hkv, D)
    cos, sin = oracle.rope_tables(np.array([c["pos"]]), D, 1e6)            # [1, D]
    q = oracle.rms_norm(qkv[:, :hq], c["qw"], eps)
    k = oracle.rms_norm(qkv[:, hq:hq + hkv], c["kw"], eps)
    rope = lambda t: oracle.apply_rope(t[:, :, None, :], cos, sin)[:, :, 0, :]  # noqa: E731   [mb, heads, D]
    return h1, act, h2, x2, (rope(q), rope(k), qkv[:, hq + hkv:])


def _run(c, eps, alias=False, entry="kd_decode_layer_fused"):
    mb, Ko = c["attn"].shape
    H, I = c["wo"].shape[0], c["wg"].shape[0]
    bf = lambda a: Tensor(a, dtype="bfloat16")  # noqa: E731
    t = {"attn": bf(c["attn"]), "wo": bf(c["wo"]), "h": Tensor(c["h"]), "post": bf(c["post"]),
         "wgu": bf(interleave_gate_up(c["wg"], c["wu"])), "wd": bf(c["wd"]), "next": bf(c["next"])}
    t["h2"] = t["h"] if alias else core.empty((mb, H), "float32")
    args = [None] * 10
    xf = None
    if c["hq"]:
        hq, hkv = c["hq"], c["hkv"]
        inv = Tensor(np.array([1.0 / (1e6 ** (i / (D // 2))) for i in range(D // 2)], np.float32))
        t["cos"], t["sin"] = core.empty((1, D // 2), "float32"), core.empty((1, D // 2), "float32")
        t["pos"] = Tensor(np.array([c["pos"]], np.int32))
        lib.call("kd_rope_table", _r(inv), _r(t["pos"]), 0, 1, _r(t["cos"]), _r(t["sin"]))
        t["kc"] = Tensor(np.full((mb + 1, hkv, c["max_s"], D), 7.0, np.float32), dtype="bfloat16")   # one spare sequence slot
        t["vc"] = Tensor(np.full((mb + 1, hkv, c["max_s"], D), 7.0, np.float32), dtype="bfloat16")
        t["q"] = core.empty((mb, 1, hq, D), "bfloat16")
        t["wq"], t["qw"], t["kw"] = bf(c["wq"]), bf(c["qw"]), bf(c["kw"])
        args = [t["wq"], t["qw"], t["kw"], t["cos"], t["sin"], t["pos"], t["kc"], t["vc"], None, t["q"]]
    else:
        xf = t["xf"] = core.empty((mb, H), "bfloat16")
    t["call"] = lambda: lib.call(entry, _r(t["attn"]), _r(t["wo"]), _r(t["h"]), _r(t["post"]), _r(t["wgu"]),
                                 _r(t["wd"]), _r(t["next"]), ctypes.c_float(eps), *[_r(a) for a in args], _r(t["h2"]), _r(xf))
    t["call"]()
    return t


def _close(got, ref, rel, what):
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    bound = rel * np.abs(ref).max()
    assert (err <= np.abs(ref) * 2.0 ** -7 + bound).all(), f"{what}: worst {err.max():.3e}, bound {bound:.3e}"


@pytest.mark.parametrize("mb,H,Ko,I,hq,hkv", [
    (32, 1024, 2048, 3072, 16, 8),     # Qwen3-0.6B, the benchmark's decode batch
    (4, 1024, 2048, 3072, 16, 8),      # the batch of one rank when 32 sequences are spread over 8 GPUs
    (5, 1024, 2048, 3072, 16, 8),      # ragged batch: padded sequence columns
    (1, 256, 128, 512, 1, 1),          # one sequence, single-split phases
    (48, 512, 320, 1056, 0, 0),        # after the last layer (x_final), 64-column accumulators, odd tile counts
    (8, 2560, 4096, 9728, 32, 8),      # Qwen3-4B widths: more units than SMs in the split-K phases
    (128, 2560, 4096, 9728, 4, 1),     # largest batch the kernel takes, the head counts of one rank of eight
])
def test_fused_layer_matches_the_unfused_oracle(backend, oracle, mb, H, Ko, I, hq, hkv):
    eps = 1e-6
    c = _case(mb, H, Ko, I, hq, hkv, f"{mb}-{H}")
    h1, act, h2, x2, qkv = _oracle(oracle, c, eps)
    lib.call("kd_debug_fill_scratch", 0xFF)        # NaN patterns: a slot that is read before it is written shows
    t = _run(c, eps)
    backend.synchronize()
    # h2 sums up to 9728 products of bf16 activations that were rounded at another point than the
    # oracle's (bf16(h1 * w) scaled afterwards, against bf16(h1 * rs * w)): near-ties fall differently
    _close(t["h2"].dataAsync(), h2, 4e-3, "h2")
    if not hq:
        _close(t["xf"].dataAsync(), x2, 4e-3, "x_final")
        return
    q, k, v = qkv
    pos = c["pos"]
    kc, vc = t["kc"].dataAsync(), t["vc"].dataAsync()
    _close(t["q"].dataAsync()[:, 0], q, 6e-3, "q")
    _close(kc[:mb, :, pos], k, 6e-3, "k row")
    _close(vc[:mb, :, pos], v, 6e-3, "v row")
    # nothing else in the caches moved: other positions and the spare sequence slot keep their fill
    kc[:mb, :, pos] = 7.0
    vc[:mb, :, pos] = 7.0
    assert (kc == 7.0).all() and (vc == 7.0).all()


def test_fused_layer_is_repeatable_in_place_and_close_to_the_chain_kernel(backend, oracle):
    eps, mb, H, Ko, I, hq, hkv = 1e-6, 32, 1024, 2048, 3072, 16, 8
    c = _case(mb, H, Ko, I, hq, hkv, "rep")
    t = _run(c, eps)
    first = {k: t[k].dataAsync().copy() for k in ("h2", "q", "kc", "vc")}
    for _ in range(4):
        t["call"]()
    for k, v in first.items():
        assert np.array_equal(t[k].dataAsync(), v), f"{k} changed between launches"
    # in place: resid_out is resid_in
    t2 = _run(c, eps, alias=True)
    assert np.array_equal(t2["h"].dataAsync(), first["h2"])
    # the six-phase chain kernel on the same operands: same h2 up to the split-K summation order and
    # the place where the RMSNorm scale is applied
    s = ctypes.c_int(0)
    lib.call("kd_decode_layer_chain_splits", ctypes.c_int64((hq + 2 * hkv) * D), ctypes.c_int64(H), ctypes.byref(s))
    h1, h2 = core.empty((mb, H), "float32"), core.empty((mb, H), "float32")
    x, act = core.empty((mb, H), "bfloat16"), core.empty((mb, I), "bfloat16")
    qp = core.empty((s.value, mb, (hq + 2 * hkv) * D), "float32")
    lib.call("kd_decode_layer_chain", _r(t["attn"]), _r(t["wo"]), _r(t["h"]), _r(t["post"]), _r(t["wgu"]), _r(t["wd"]),
             _r(t["next"]), ctypes.c_float(eps), _r(t["wq"]), _r(h1), _r(h2), _r(x), _r(act), _r(qp))
    _close(first["h2"], h2.dataAsync(), 2e-3, "h2 against the chain kernel")


def test_fused_layer_reports_a_cache_row_outside_the_cache_and_checks_arguments(backend, oracle):
    eps = 1e-6
    c = _case(2, 256, 128, 512, 1, 1, "bad", max_s=8, pos=8)        # row 8 of an 8-row cache
    t = _run(c, eps)
    with pytest.raises(lib.KandleCudaError) as e:
        backend.synchronize()
    assert e.value.status == 6 and "102" in str(e.value)
    assert (t["kc"].dataAsync() == 7.0).all()                         # nothing was written
    c = _case(2, 256, 128, 512, 1, 1, "ok", max_s=8, pos=7)
    t = _run(c, eps)                                                  # the context is still usable
    backend.synchronize()
    assert not (t["kc"].dataAsync()[:2, :, 7] == 7.0).all()
    with pytest.raises(lib.KandleCudaError):                          # QKV weights without caches
        lib.call("kd_decode_layer_fused", _r(t["attn"]), _r(t["wo"]), _r(t["h"]), _r(t["post"]), _r(t["wgu"]), _r(t["wd"]),
                 _r(t["next"]), ctypes.c_float(eps), _r(t["wq"]), None, None, None, None, None, None, None, None, None, _r(t["h2"]), None)
    with pytest.raises(lib.KandleCudaError):                          # last-layer form without x_final
        lib.call("kd_decode_layer_fused", _r(t["attn"]), _r(t["wo"]), _r(t["h"]), _r(t["post"]), _r(t["wgu"]), _r(t["wd"]),
                 _r(t["next"]), ctypes.c_float(eps), None, None, None, None, None, None, None, None, None, None, _r(t["h2"]), None)


def test_tensor_parallel_form_with_stand_in_peers_matches_the_plain_kernel_then_times_out(backend, oracle):
    """One GPU: this process is rank 0 of 4 whose peers are local buffers.  Launch 1 finds their
    flags set and their partial sums zero, so it must give what the plain kernel gives (up to the
    order in which a sequence's sum of squares is added up: that epilogue is organised differently); launch 2
    waits for peers that never answer, gives up after its bound (error 531) and leaves the
    context usable."""
    eps, mb, H, Ko, I, hq, hkv = 1e-6, 8, 2560, 2048, 2432, 8, 2        # one rank's share of the Qwen3-4B layer on 4 GPUs
    c = _case(mb, H, Ko, I, hq, hkv, "tp")
    plain = _run(c, eps)
    backend.synchronize()
    want = {k: plain[k].dataAsync().copy() for k in ("h2", "q", "kc", "vc")}
    lib.call("kd_p2p_selftest_silent_peers", 4, ctypes.c_uint32(20_000_000), ctypes.c_uint32(1))
    try:
        t = _run(c, eps, entry="kd_decode_layer_fused_tp")
        backend.synchronize()
        for k, v in want.items():
            _close(t[k].dataAsync(), v, 1e-3, f"{k} (tensor-parallel form against the plain kernel)")
        t["call"]()                                                    # tag 2: nobody answers
        with pytest.raises(lib.KandleCudaError) as e:
            backend.synchronize()
        assert e.value.status == 6 and "531" in str(e.value)
    finally:
        lib.call("kd_p2p_disconnect")
    again = _run(c, eps)                                               # the context and the kernel still work
    backend.synchronize()
    assert np.array_equal(again["h2"].dataAsync(), want["h2"])
    with pytest.raises(lib.KandleCudaError):                           # no peers connected
        _run(c, eps, entry="kd_decode_layer_fused_tp")
