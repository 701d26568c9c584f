"""Kernel registration for `CudaBackend`: one function per dispatch key, with the signatures the
reference's dispatch handlers call (what `registerWebGPUKernels` does for the WebGPU backend,
packages/backend-webgpu/src/kernels/index.ts:36-90).

Signatures (all synchronous, enqueue-only, raise on misuse):
  iterator keys      fn(iter: TensorIterator) -> None
  matmul             fn(cfg: MatmulDispatchResult, a, b) -> None           (writes cfg.output)
  rms_norm, layer_norm, softmax
                     fn(inputs: [x], params: dict) -> handle               (kernel allocates)
  index_select       fn(self, index, {"dim": d}, output) -> None
  flash_attention    fn(q, k, v, out, scale, isCausal) -> None
  conv1d             fn(cfg: ConvDispatchResult, input, weight, bias=None) -> handle
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

from . import lib
from .lib import POINTWISE_OPS, kd_matmul_cfg


def _ref(h):
    return ctypes.byref(h.c()) if h is not None else None


@dataclass
class TensorIterator:
    """The part of ITensorIterator the map kernels read (packages/types/src/tensor.ts:395-569):
    pre-allocated output, inputs already broadcast-compatible with it, scalar arguments."""
    inputs: list
    outputs: list
    scalars: dict = field(default_factory=dict)

    def input(self, i: int = 0):
        return self.inputs[i]

    def output(self, i: int = 0):
        return self.outputs[i]

    def getScalarArgs(self) -> dict:
        return self.scalars


@dataclass
class MatmulDispatchResult:
    """packages/core/src/dispatch/matmulOps.ts:32-125 (fields the kernel reads)."""
    variant: str
    output: object
    M: int
    K: int
    N: int
    batchShape: tuple
    transposeA: bool = False
    transposeB: bool = False
    alpha: float = 1.0
    beta: float = 0.0
    inputC: object = None

    @property
    def batchSize(self) -> int:
        n = 1
        for b in self.batchShape:
            n *= b
        return n


@dataclass
class ConvDispatchResult:
    """packages/core/src/dispatch/handlers/window.ts:45-87 (fields the conv1d kernel reads)."""
    stride: int
    padding: int
    outputShape: tuple
    dtype: str


def _pointwise(key: str):
    op = POINTWISE_OPS[key]

    def fn(it: TensorIterator) -> None:
        a = it.input(0)
        b = it.inputs[1] if len(it.inputs) > 1 else None
        sc = it.getScalarArgs()
        scalar = float(sc.get("alpha", sc.get("scalar", sc.get("other", 1.0))))
        lib.call("kd_pointwise", op, _ref(a), _ref(b), ctypes.c_float(scalar), _ref(it.output()))

    return fn


def _copy(it: TensorIterator) -> None:
    lib.call("kd_copy", _ref(it.output()), _ref(it.input(0)))


def _fill(value):
    def fn(it: TensorIterator) -> None:
        v = it.getScalarArgs().get("fillValue", value) if value is None else value
        lib.call("kd_fill", _ref(it.output()), ctypes.c_double(float(v)))
    return fn


def _empty(it: TensorIterator) -> None:
    return None


def _arange(it: TensorIterator) -> None:
    s = it.getScalarArgs()
    lib.call("kd_arange", _ref(it.output()), ctypes.c_double(float(s.get("start", 0))),
             ctypes.c_double(float(s.get("step", 1))))


class RandomState:
    """Global generator state the random kernels draw from (packages/types/src/random.ts:20-104):
    a 64-bit seed that becomes the Philox key and an offset that advances by the number of Philox
    calls each operation consumes, so that consecutive operations give different numbers."""
    seed = 0
    offset = 0

    @classmethod
    def manual_seed(cls, seed: int) -> None:
        cls.seed, cls.offset = int(seed) & 0xFFFFFFFFFFFFFFFF, 0

    @classmethod
    def consume_offset(cls, count: int) -> int:
        cur = cls.offset
        cls.offset += int(count)
        return cur


def _randn(it: TensorIterator) -> None:
    """Key `randn`: N(0,1) into the pre-allocated output (executor.ts:31-49: numel / 2 Philox calls)."""
    out = it.output()
    base = RandomState.consume_offset((out.numel + 1) // 2)
    lib.call("kd_randn", _ref(out), ctypes.c_uint64(RandomState.seed), ctypes.c_uint32(base & 0xFFFFFFFF), ctypes.c_float(0.0),
             ctypes.c_float(1.0), 0, 0, 0)


def _argmax(it: TensorIterator) -> None:
    lib.call("kd_argmax", _ref(it.input(0)), _ref(it.output()))


def _matmul(cfg: MatmulDispatchResult, a, b) -> None:
    c = kd_matmul_cfg()
    c.M, c.N, c.K = cfg.M, cfg.N, cfg.K
    c.transpose_a, c.transpose_b = int(cfg.transposeA), int(cfg.transposeB)
    c.alpha, c.beta = float(cfg.alpha), float(cfg.beta)
    c.has_c = int(cfg.inputC is not None)
    lib.call("kd_matmul", ctypes.byref(c), _ref(a), _ref(b), _ref(cfg.inputC), _ref(cfg.output))


def _alloc_like(x, out):
    from .backend import CudaBackend
    if out is not None:
        return out
    return CudaBackend.instance().createTensorHandle(x.shape, x.dtype)


def _rms_norm(inputs, params):
    x = inputs[0]
    out = _alloc_like(x, params.get("out"))
    lib.call("kd_rms_norm", _ref(x), _ref(params.get("weight")), ctypes.c_float(params.get("eps", 1e-5)), _ref(out))
    return out


def _layer_norm(inputs, params):
    x = inputs[0]
    out = _alloc_like(x, params.get("out"))
    lib.call("kd_layer_norm", _ref(x), _ref(params.get("weight")), _ref(params.get("bias")),
             ctypes.c_float(params.get("eps", 1e-5)), _ref(out))
    return out


def _softmax(inputs, params):
    x = inputs[0]
    dim = params.get("dim", -1)
    if dim not in (-1, len(x.shape) - 1):
        raise lib.KandleCudaError(5, "softmax is implemented over the last dimension only")
    out = _alloc_like(x, params.get("out"))
    lib.call("kd_softmax", _ref(x), _ref(out))
    return out


def _index_select(self_h, index, params, output) -> None:
    lib.call("kd_index_select", _ref(self_h), _ref(index), int(params.get("dim", 0)), _ref(output))


def _flash_attention(q, k, v, out, scale: float, isCausal: bool) -> None:
    lib.call("kd_flash_attention", _ref(q), _ref(k), _ref(v), _ref(out), ctypes.c_float(scale), int(bool(isCausal)))


def _conv1d(cfg: ConvDispatchResult, inp, weight, bias=None):
    from .backend import CudaBackend
    out = CudaBackend.instance().createTensorHandle(cfg.outputShape, cfg.dtype)
    lib.call("kd_conv1d", _ref(inp), _ref(weight), _ref(bias), int(cfg.stride), int(cfg.padding), _ref(out))
    return out


def register_cuda_kernels(ops) -> None:
    for key in POINTWISE_OPS:
        ops.register(key, _pointwise(key))
    for key in ("copy", "contiguous", "copy_", "cast", "clone"):
        ops.register(key, _copy)
    ops.register("zeros", _fill(0.0))
    ops.register("ones", _fill(1.0))
    ops.register("full", _fill(None))
    ops.register("empty", _empty)
    ops.register("arange", _arange)
    ops.register("randn", _randn)
    ops.register("argmax", _argmax)
    ops.register("matmul", _matmul)
    ops.register("rms_norm", _rms_norm)
    ops.register("layer_norm", _layer_norm)
    ops.register("softmax", _softmax)
    ops.register("index_select", _index_select)
    ops.register("flash_attention", _flash_attention)
    ops.register("conv1d", _conv1d)
