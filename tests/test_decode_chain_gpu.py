"""GPU parity of kd_decode_layer_chain (o_proj -> add+RMSNorm -> gate/up SiLU*up -> down ->
add+RMSNorm -> next QKV as one persistent kernel) against the oracle's unfused operator sequence
(what packages/model-utils/src/qwen3/decoder_layer.ts:191-241 computes for one new token) and
against the library's own separate kernels."""
import ctypes

import numpy as np
import pytest

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor
from kandle_b200.engine import interleave_gate_up

pytestmark = pytest.mark.gpu


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


def _splits(n, k):
    s = ctypes.c_int(0)
    lib.call("kd_decode_layer_chain_splits", ctypes.c_int64(n), ctypes.c_int64(k), ctypes.byref(s))
    return s.value


def _rb(a):
    return lib.round_to_bf16(np.ascontiguousarray(a, dtype=np.float32))


def _case(mb, H, Ko, I, Nq, seed):
    n = lambda name, shape, std=1.0: synth.normal(f"{name}{seed}", shape, std)  # noqa: E731
    c = {
        "attn": _rb(n("attn", (mb, Ko))), "wo": _rb(n("wo", (H, Ko), 0.03)), "h": n("h", (mb, H)),
        "post": _rb(1.0 + n("post", (H,), 0.1)), "wg": _rb(n("wg", (I, H), 0.03)), "wu": _rb(n("wu", (I, H), 0.03)),
        "wd": _rb(n("wd", (H, I), 0.03)), "next": _rb(1.0 + n("next", (H,), 0.1)),
        "wq": _rb(n("wq", (Nq, H), 0.03)) if Nq else None,
    }
    return c


def _oracle_chain(oracle, c, eps):
    h1 = c["h"] + oracle.linear(c["attn"], c["wo"])
    x = _rb(oracle.rms_norm(h1, c["post"], eps))
    g, u = oracle.linear(x, c["wg"]), oracle.linear(x, c["wu"])
    act = _rb(oracle.unary("silu", g) * u)
    h2 = h1 + oracle.linear(act, c["wd"])
    x2 = _rb(oracle.rms_norm(h2, c["next"], eps))
    qkv = oracle.linear(x2, c["wq"]) if c["wq"] is not None else None
    return h1, act, h2, x2, qkv


def _run_chain(c, eps, alias=True):
    mb, Ko = c["attn"].shape
    H, I = c["wo"].shape[0], c["wg"].shape[0]
    bf = lambda a: Tensor(a, dtype="bfloat16")  # noqa: E731
    t = {
        "attn": bf(c["attn"]), "wo": bf(c["wo"]), "h": Tensor(c["h"]), "post": bf(c["post"]),
        "wgu": bf(interleave_gate_up(c["wg"], c["wu"])), "wd": bf(c["wd"]), "next": bf(c["next"]),
        "h1": core.empty((mb, H), "float32"), "x": core.empty((mb, H), "bfloat16"), "act": core.empty((mb, I), "bfloat16"),
    }
    t["h2"] = t["h"] if alias else core.empty((mb, H), "float32")
    wq = qp = None
    if c["wq"] is not None:
        wq = t["wq"] = bf(c["wq"])
        qp = t["qp"] = core.empty((_splits(c["wq"].shape[0], H), mb, c["wq"].shape[0]), "float32")
    lib.call("kd_decode_layer_chain", _r(t["attn"]), _r(t["wo"]), _r(t["h"]), _r(t["post"]), _r(t["wgu"]), _r(t["wd"]),
             _r(t["next"]), ctypes.c_float(eps), _r(wq), _r(t["h1"]), _r(t["h2"]), _r(t["x"]), _r(t["act"]), _r(qp))
    return t


def _close(got, ref, rel, what):
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    bound = rel * np.abs(ref).max()
    assert (err <= np.abs(ref) * 2.0 ** -7 + bound).all(), f"{what}: worst {err.max():.3e}, bound {bound:.3e}"


@pytest.mark.parametrize("mb,H,Ko,I,Nq", [
    (32, 1024, 2048, 3072, 4096),      # Qwen3-0.6B, the benchmark's decode batch
    (5, 1024, 2048, 3072, 4096),       # ragged batch: padded token columns
    (1, 256, 128, 512, 384),           # one sequence, one k-block splits
    (48, 512, 320, 1056, 0),           # last layer (no QKV phase), 64-row activation box, odd tile counts
    (128, 2560, 4096, 9728, 6144),     # Qwen3-4B widths at the largest batch the kernel takes
])
def test_chain_matches_the_unfused_oracle(backend, oracle, mb, H, Ko, I, Nq):
    eps = 1e-6
    c = _case(mb, H, Ko, I, Nq, f"{mb}-{H}")
    h1, act, h2, x2, qkv = _oracle_chain(oracle, c, eps)
    t = _run_chain(c, eps, alias=False)
    backend.synchronize()
    # fp32 quantities: accumulation order only.  bf16 quantities: one rounding step of their own,
    # plus the effect of bf16 ties in the activations upstream of them.
    _close(t["h1"].dataAsync(), h1, 1e-5, "h1")
    _close(t["act"].dataAsync(), act, 4e-3, "act")
    _close(t["h2"].dataAsync(), h2, 2e-3, "h2")
    _close(t["x"].dataAsync(), x2, 4e-3, "x")
    if qkv is not None:
        _close(t["qp"].dataAsync().sum(0), qkv, 4e-3, "qkv")


def test_chain_equals_the_separate_kernels_and_is_repeatable(backend):
    """Same operands through the six separate kernels: identical bf16 activations up to the
    different split-K summation order, and bit-identical results launch after launch (no atomics
    on data)."""
    eps, mb, H, Ko, I, Nq = 1e-6, 32, 1024, 2048, 3072, 4096
    c = _case(mb, H, Ko, I, Nq, "sep")
    t = _run_chain(c, eps, alias=False)
    first = {k: t[k].dataAsync().copy() for k in ("h1", "act", "h2", "x", "qp")}
    for _ in range(3):
        lib.call("kd_decode_layer_chain", _r(t["attn"]), _r(t["wo"]), _r(t["h"]), _r(t["post"]), _r(t["wgu"]), _r(t["wd"]),
                 _r(t["next"]), ctypes.c_float(eps), _r(t["wq"]), _r(t["h1"]), _r(t["h2"]), _r(t["x"]), _r(t["act"]), _r(t["qp"]))
    for k, v in first.items():
        assert np.array_equal(t[k].dataAsync(), v), f"{k} changed between launches"
    # separate kernels
    op = core.empty((4, mb, H), "float32")
    lib.call("kd_linear_bf16_skinny", _r(t["attn"]), _r(t["wo"]), 0, _r(op))
    h1, x = core.empty((mb, H), "float32"), core.empty((mb, H), "bfloat16")
    e = ctypes.c_float(eps)
    lib.call("kd_add_rmsnorm", _r(op), _r(t["h"]), _r(t["post"]), e, _r(h1), _r(x))
    act = core.empty((mb, I), "bfloat16")
    lib.call("kd_linear_bf16_skinny", _r(x), _r(t["wgu"]), 2, _r(act))
    dp = core.empty((5, mb, H), "float32")
    lib.call("kd_linear_bf16_skinny", _r(act), _r(t["wd"]), 0, _r(dp))
    h2, x2 = core.empty((mb, H), "float32"), core.empty((mb, H), "bfloat16")
    lib.call("kd_add_rmsnorm", _r(dp), _r(h1), _r(t["next"]), e, _r(h2), _r(x2))
    _close(first["h1"], h1.dataAsync(), 1e-5, "h1")
    _close(first["h2"], h2.dataAsync(), 2e-3, "h2")
    _close(first["x"], x2.dataAsync(), 4e-3, "x")
    assert (first["act"] == act.dataAsync()).mean() > 0.99


def test_chain_in_place_residual_and_argument_checks(backend, oracle):
    eps = 1e-6
    c = _case(8, 256, 128, 512, 384, "inplace")
    _, _, h2, x2, _ = _oracle_chain(oracle, c, eps)
    t = _run_chain(c, eps, alias=True)      # resid_out is resid_in
    _close(t["h"].dataAsync(), h2, 2e-3, "h (in place)")
    _close(t["x"].dataAsync(), x2, 4e-3, "x")
    bad = core.empty((8, 256), "bfloat16")   # residual must be fp32
    with pytest.raises(lib.KandleCudaError):
        lib.call("kd_decode_layer_chain", _r(t["attn"]), _r(t["wo"]), _r(bad), _r(t["post"]), _r(t["wgu"]), _r(t["wd"]),
                 _r(t["next"]), ctypes.c_float(eps), None, _r(t["h1"]), _r(t["h2"]), _r(t["x"]), _r(t["act"]), None)
    with pytest.raises(lib.KandleCudaError):   # QKV weights without a place for the partial sums
        lib.call("kd_decode_layer_chain", _r(t["attn"]), _r(t["wo"]), _r(t["h"]), _r(t["post"]), _r(t["wgu"]), _r(t["wd"]),
                 _r(t["next"]), ctypes.c_float(eps), _r(t["wq"]), _r(t["h1"]), _r(t["h2"]), _r(t["x"]), _r(t["act"]), None)
