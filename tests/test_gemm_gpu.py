"""GPU parity of the tcgen05 bf16 GEMM (`linear` on the tensor cores) against the CPU oracle.

Inputs are rounded to bf16 once and the oracle computes in fp32 on the rounded values, so the only
differences are accumulation order and the single bf16 rounding of the output:
|err| <= 2^-8 * |ref| + small absolute slack."""
import ctypes

import numpy as np
import pytest

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor

pytestmark = pytest.mark.gpu


def bf16_close(got, ref, extra=1e-3):
    ref = ref.astype(np.float64)
    err = np.abs(got.astype(np.float64) - ref)
    bound = np.abs(ref) * 2.0 ** -8 + extra * np.abs(ref).max()
    bad = err > bound
    assert not bad.any(), f"{bad.sum()} of {bad.size} outside the bf16 bound; worst {err.max():.3e} (ref max {np.abs(ref).max():.3e})"


def _linear_bf16(x, w, resid=None, epilogue=0, out_dtype="bfloat16"):
    tx, tw = Tensor(x, dtype="bfloat16"), Tensor(w, dtype="bfloat16")
    n_out = w.shape[0] // 2 if epilogue == 2 else w.shape[0]
    out = core.empty(x.shape[:-1] + (n_out,), out_dtype)
    tr = Tensor(resid, dtype="bfloat16") if resid is not None else None
    lib.call("kd_linear_bf16", ctypes.byref(tx._handle.c()), ctypes.byref(tw._handle.c()),
             ctypes.byref(tr._handle.c()) if tr is not None else None, epilogue, ctypes.byref(out._handle.c()))
    return out.dataAsync()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 128, 128), (256, 512, 1024), (300, 1000, 264), (1, 256, 64),
                                   (77, 64, 72), (2048, 3072, 1024), (515, 2048, 3072), (130, 8, 40)])
def test_linear_bf16_matches_oracle(backend, oracle, m, n, k):
    x, w = lib.round_to_bf16(synth.normal("x", (m, k))), lib.round_to_bf16(synth.normal("w", (n, k), 0.05))
    ref = oracle.linear(x, w)
    bf16_close(_linear_bf16(x, w), ref)
    got32 = _linear_bf16(x, w, out_dtype="float32")
    assert np.abs(got32 - ref).max() <= 1e-4 * np.abs(ref).max()     # fp32 output: accumulation order only


def test_linear_bf16_residual_epilogue(backend, oracle):
    x, w = lib.round_to_bf16(synth.normal("x", (200, 2048))), lib.round_to_bf16(synth.normal("w", (1024, 2048), 0.02))
    r = lib.round_to_bf16(synth.normal("r", (200, 1024)))
    bf16_close(_linear_bf16(x, w, r, 1), oracle.add(r, oracle.linear(x, w)))


def test_linear_bf16_swiglu_epilogue(backend, oracle):
    """Fused gate/up weight: per 32-row block, 16 gate rows then the 16 matching up rows."""
    K, I = 1024, 768
    x = lib.round_to_bf16(synth.normal("x", (150, K)))
    wg, wu = lib.round_to_bf16(synth.normal("wg", (I, K), 0.03)), lib.round_to_bf16(synth.normal("wu", (I, K), 0.03))
    fused = np.concatenate([np.concatenate([wg[i:i + 16], wu[i:i + 16]]) for i in range(0, I, 16)])
    ref = oracle.mul(oracle.unary("silu", oracle.linear(x, wg)), oracle.linear(x, wu))
    bf16_close(_linear_bf16(x, fused, None, 2), ref, 2e-3)


def test_matmul_key_routes_bf16_to_tensor_cores(backend, oracle):
    """The registry key `matmul` with bf16 operands (linear and the tied lm_head's strided view)."""
    h, e = lib.round_to_bf16(synth.normal("h", (2, 40, 256))), lib.round_to_bf16(synth.normal("e", (1000, 256), 0.05))
    th, te = Tensor(h, dtype="bfloat16"), Tensor(e, dtype="bfloat16")
    before = backend.launch_count(reset=True)
    y = core.linear(th, te)
    assert y.dtype == "bfloat16" and y.shape == (2, 40, 1000)
    bf16_close(y.dataAsync(), oracle.linear(h, e))
    et = te.transpose(0, 1)
    bf16_close(core.matmul(th, et).dataAsync(), oracle.linear(h, e))
    # an operand layout the tensor-core path does not take still works (CUDA-core kernel)
    a = lib.round_to_bf16(synth.normal("a", (9, 7)))
    b = lib.round_to_bf16(synth.normal("b", (7, 5)))
    bf16_close(core.matmul(Tensor(a, dtype="bfloat16"), Tensor(b, dtype="bfloat16")).dataAsync(), a @ b)


def test_linear_bf16_rejects_bad_arguments(backend):
    x, w = Tensor(synth.normal("x", (4, 64))), Tensor(synth.normal("w", (8, 64)), dtype="bfloat16")
    out = core.empty((4, 8), "bfloat16")
    with pytest.raises(lib.KandleCudaError):
        lib.call("kd_linear_bf16", ctypes.byref(x._handle.c()), ctypes.byref(w._handle.c()), None, 0, ctypes.byref(out._handle.c()))
