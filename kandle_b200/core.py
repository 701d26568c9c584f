"""Host-side mirror of the slice of `@kandle/core` that sits between the models and the backend
boundary: the `env` registry, the `Tensor` wrapper with its view operations, and the dispatch
handlers that turn user-level ops into backend kernel calls.

Reference counterparts: `env` (packages/core/src/env.ts:3-43), `Tensor`
(packages/core/src/tensor.ts), iterator handler (dispatch/handlers/iterator.ts:34-231 with
TensorIterator.build, dispatch/TensorIterator.ts:191-285), `dispatchMatmul`
(dispatch/matmulOps.ts:408-496), composite handler for `linear`, `embedding` and
`scaled_dot_product_attention` (dispatch/handlers/composite.ts:55-77,149-245,247-348), normalize
handler (dispatch/handlers/normalize.ts:46-95), gather handler (dispatch/handlers/gather.ts:97-137).
Every op looks the backend up through `env` and calls `backend.operators.find(key)` exactly where
the reference does, so the sequence of backend calls for a model is the reference's sequence.
"""
from __future__ import annotations

import math
from typing import Sequence

import numpy as np

from .backend import CudaBackend, CudaTensorHandle, contiguous_strides
from .kernels import ConvDispatchResult, MatmulDispatchResult, TensorIterator


class _Env:
    def __init__(self):
        self._backends = {}
        self._default = None

    def setBackend(self, backend) -> None:
        self._backends[backend.name] = backend

    def getBackend(self, device: str):
        if device not in self._backends:
            raise RuntimeError(f"No backend registered for device '{device}'")
        return self._backends[device]

    def setDefaultDevice(self, device: str) -> None:
        if device not in self._backends:
            raise RuntimeError(f"No backend registered for device '{device}'")
        self._default = device

    def getDefaultDevice(self) -> str:
        if self._default is None:
            raise RuntimeError("no default device set")
        return self._default


env = _Env()


def init(device_ordinal: int = 0) -> CudaBackend:
    """Creates the CUDA backend and registers it as default device, the sequence the reference's
    playground runs for WebGPU (playground-node/src/init.ts:25-28)."""
    be = CudaBackend.create(device_ordinal)
    env.setBackend(be)
    env.setDefaultDevice("cuda")
    return be


def _backend():
    return env.getBackend(env.getDefaultDevice())


def _kernel(key: str):
    fn = _backend().operators.find(key)
    if fn is None:
        raise RuntimeError(f"Kernel '{key}' not registered in backend")
    return fn


_FLOAT_RANK = {"bfloat16": 1, "float16": 1, "float32": 2}


def _promote(a: str, b: str) -> str:
    """Result dtype of a binary op (subset of packages/utils/src/dtype.ts:233-278)."""
    if a == b:
        return a
    fa, fb = a in _FLOAT_RANK, b in _FLOAT_RANK
    if fa and fb:
        if {a, b} == {"bfloat16", "float16"}:
            return "float32"
        return a if _FLOAT_RANK[a] >= _FLOAT_RANK[b] else b
    if fa:
        return a
    if fb:
        return b
    order = ["bool", "uint8", "int32", "int64"]
    return a if order.index(a) >= order.index(b) else b


def _broadcast_shape(a: Sequence[int], b: Sequence[int]) -> tuple:
    n = max(len(a), len(b))
    a = (1,) * (n - len(a)) + tuple(a)
    b = (1,) * (n - len(b)) + tuple(b)
    out = []
    for x, y in zip(a, b):
        if x == y or y == 1:
            out.append(x)
        elif x == 1:
            out.append(y)
        else:
            raise ValueError(f"shapes {a} and {b} are not broadcastable")
    return tuple(out)


def _parse_slice(spec: str, shape: Sequence[int]):
    """Python-style slice strings such as ':, :, 3:7, :' or '..., :64'
    (packages/utils/src/slice-parser.ts)."""
    parts = [p.strip() for p in spec.split(",")]
    n_explicit = sum(1 for p in parts if p != "...")
    items = []
    for p in parts:
        if p == "...":
            items.extend([slice(None)] * (len(shape) - n_explicit))
        elif ":" in p:
            f = [int(x) if x.strip() else None for x in p.split(":")]
            items.append(slice(*f))
        else:
            items.append(int(p))
    items.extend([slice(None)] * (len(shape) - len(items)))
    if len(items) != len(shape):
        raise ValueError(f"slice '{spec}' does not match rank {len(shape)}")
    return items


class Tensor:
    """Thin wrapper over a backend handle (packages/core/src/tensor.ts:8).  `Tensor(data, dtype=,
    shape=)` uploads through `backend.createTensorHandle(shape, dtype, data)` (tensor.ts:184-186)."""

    def __init__(self, data=None, *, dtype: str | None = None, shape=None, _handle: CudaTensorHandle | None = None):
        if _handle is not None:
            self._handle = _handle
            return
        arr = np.asarray(data)
        if dtype is None:
            dtype = {"float64": "float32", "float32": "float32", "int64": "int64", "int32": "int32",
                     "uint8": "uint8", "bool": "bool", "float16": "float16"}[arr.dtype.name]
        if shape is None:
            shape = arr.shape
        self._handle = _backend().createTensorHandle(tuple(shape), dtype, arr)

    # --- metadata
    @property
    def shape(self) -> tuple:
        return self._handle.shape

    @property
    def dtype(self) -> str:
        return self._handle.dtype

    @property
    def strides(self) -> tuple:
        return self._handle.strides

    @property
    def offset(self) -> int:
        return self._handle.offset

    @property
    def ndim(self) -> int:
        return len(self._handle.shape)

    @property
    def numel(self) -> int:
        return self._handle.numel

    def isContiguous(self) -> bool:
        return self._handle.isContiguous()

    def dataAsync(self) -> np.ndarray:
        return self._handle.dataAsync()

    def dispose(self) -> None:
        self._handle.dispose()

    # --- views (metadata only)
    def _view(self, shape, strides, offset) -> "Tensor":
        return Tensor(_handle=self._handle.view(shape, strides, offset))

    def view(self, *shape) -> "Tensor":
        shape = tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else tuple(shape)
        if -1 in shape:
            known = -math.prod(shape)
            shape = tuple(self.numel // known if s == -1 else s for s in shape)
        if math.prod(shape) != self.numel:
            raise ValueError(f"view shape {shape} is invalid for {self.numel} elements")
        if not self.isContiguous():
            raise ValueError("view() needs a contiguous tensor; call contiguous() first")
        return self._view(shape, contiguous_strides(shape), self.offset)

    def reshape(self, *shape) -> "Tensor":
        if self.isContiguous():
            return self.view(*shape)
        c = contiguous(self)
        out = c.view(*shape)
        c.dispose()
        return out

    def permute(self, dims: Sequence[int]) -> "Tensor":
        dims = [d % self.ndim for d in dims]
        return self._view([self.shape[d] for d in dims], [self.strides[d] for d in dims], self.offset)

    def transpose(self, d0: int, d1: int) -> "Tensor":
        dims = list(range(self.ndim))
        dims[d0], dims[d1] = dims[d1], dims[d0]
        return self.permute(dims)

    def unsqueeze(self, dim: int) -> "Tensor":
        dim = dim % (self.ndim + 1)
        shape, strides = list(self.shape), list(self.strides)
        shape.insert(dim, 1)
        strides.insert(dim, strides[dim] * self.shape[dim] if dim < self.ndim else 1)
        return self._view(shape, strides, self.offset)

    def expand(self, shape: Sequence[int]) -> "Tensor":
        shape = tuple(shape)
        pad = len(shape) - self.ndim
        old_shape = (1,) * pad + self.shape
        old_strides = (0,) * pad + self.strides
        strides = []
        for s, o, st in zip(shape, old_shape, old_strides):
            if s == o or s == -1:
                strides.append(st)
            elif o == 1:
                strides.append(0)
            else:
                raise ValueError(f"cannot expand {self.shape} to {shape}")
        shape = tuple(o if s == -1 else s for s, o in zip(shape, old_shape))
        return self._view(shape, strides, self.offset)

    def slice(self, spec) -> "Tensor":
        items = _parse_slice(spec, self.shape) if isinstance(spec, str) else list(spec)
        shape, strides, offset = [], [], self.offset
        for it, n, st in zip(items, self.shape, self.strides):
            if isinstance(it, int):
                idx = it + n if it < 0 else it
                if idx < 0 or idx >= n:     # the reference throws (dispatch/handlers/shape.ts:511-518), it never wraps
                    raise IndexError(f"select: index {it} out of range for dim {len(shape)} with size {n}")
                offset += idx * st
            else:
                a, b, step = it.indices(n)
                if step <= 0:
                    raise ValueError("slice step must be positive")
                shape.append(max(0, (b - a + step - 1) // step))
                strides.append(st * step)
                offset += a * st
        return self._view(shape, strides, offset)

    def select(self, dim: int, index: int) -> "Tensor":
        """packages/core/src/dispatch/handlers/shape.ts:500-540, with its two range errors."""
        nd = dim + self.ndim if dim < 0 else dim
        if nd < 0 or nd >= self.ndim:
            raise IndexError(f"select: dim {dim} out of range for tensor with {self.ndim} dimensions")
        n = self.shape[nd]
        idx = index + n if index < 0 else index
        if idx < 0 or idx >= n:
            raise IndexError(f"select: index {index} out of range for dim {dim} with size {n}")
        items = [slice(None)] * self.ndim
        items[nd] = int(idx)
        return self.slice(items)

    def contiguous(self) -> "Tensor":
        return contiguous(self)

    def clone(self) -> "Tensor":
        return _copy_like("clone", self, self.dtype)

    def to(self, dtype: str) -> "Tensor":
        return cast(self, dtype)


# ----------------------------------------------------------------------------- iterator ops
def _new(shape, dtype) -> CudaTensorHandle:
    return _backend().createTensorHandle(tuple(shape), dtype)


def _binary(key: str, a: Tensor, b, scalars=None) -> Tensor:
    if not isinstance(b, Tensor):
        if key == "mul":
            return _unary("mul_scalar", a, {"scalar": float(b)})
        # a Python scalar takes the tensor's dtype when it can (an int next to an integer tensor stays
        # integer); a float next to an integer tensor promotes to float32
        if a.dtype not in _FLOAT_RANK and float(b) == int(b) and not isinstance(b, float):
            b = Tensor(np.asarray(b).reshape(()), dtype=a.dtype)
        else:
            b = Tensor(np.asarray(b, dtype=np.float32).reshape(()), dtype="float32")
    shape = _broadcast_shape(a.shape, b.shape)
    out = _new(shape, _promote(a.dtype, b.dtype))
    _kernel(key)(TensorIterator([a._handle, b._handle], [out], scalars or {}))
    return Tensor(_handle=out)


def _unary(key: str, a: Tensor, scalars=None) -> Tensor:
    # neg / abs keep an integer dtype; the transcendental keys promote integers to float32
    keep = a.dtype in _FLOAT_RANK or key in ("neg", "abs")
    out = _new(a.shape, a.dtype if keep else "float32")
    _kernel(key)(TensorIterator([a._handle], [out], scalars or {}))
    return Tensor(_handle=out)


def add(a: Tensor, b, alpha: float = 1.0) -> Tensor:
    return _binary("add", a, b, {"alpha": alpha})


def sub(a: Tensor, b, alpha: float = 1.0) -> Tensor:
    return _binary("sub", a, b, {"alpha": alpha})


def mul(a: Tensor, b) -> Tensor:
    return _binary("mul", a, b)


def div(a: Tensor, b) -> Tensor:
    return _binary("div", a, b)


def maximum(a: Tensor, b) -> Tensor:
    return _binary("maximum", a, b)


def neg(a: Tensor) -> Tensor:
    return _unary("neg", a)


def cos(a: Tensor) -> Tensor:
    return _unary("cos", a)


def sin(a: Tensor) -> Tensor:
    return _unary("sin", a)


def silu(a: Tensor) -> Tensor:
    return _unary("silu", a)


def gelu(a: Tensor, approximate: str = "none") -> Tensor:
    # `approximate` is accepted and ignored, as in the reference (always the tanh form).
    return _unary("gelu", a)


def abs(a: Tensor) -> Tensor:  # noqa: A001 - mirrors the reference's op name
    return _unary("abs", a)


def tanh(a: Tensor) -> Tensor:
    return _unary("tanh", a)


def sigmoid(a: Tensor) -> Tensor:
    return _unary("sigmoid", a)


def _copy_like(key: str, a: Tensor, dtype: str) -> Tensor:
    out = _new(a.shape, dtype)
    _kernel(key)(TensorIterator([a._handle], [out]))
    return Tensor(_handle=out)


def contiguous(a: Tensor) -> Tensor:
    """New contiguous tensor (the reference returns a fresh tensor even when already contiguous)."""
    return _copy_like("contiguous", a, a.dtype)


def cast(a: Tensor, dtype: str) -> Tensor:
    return _copy_like("cast", a, dtype)


def copy_(dst: Tensor, src: Tensor) -> Tensor:
    """In-place strided copy (`internal.copy_`, dispatch/handlers/copy.ts:286-298): shapes must
    match after broadcasting src."""
    if _broadcast_shape(dst.shape, src.shape) != tuple(dst.shape):
        raise ValueError(f"copy_: source shape {src.shape} does not broadcast to {dst.shape}")
    _kernel("copy_")(TensorIterator([src._handle], [dst._handle]))
    return dst


def zeros(shape, dtype: str = "float32") -> Tensor:
    out = _new(shape, dtype)
    _kernel("zeros")(TensorIterator([], [out]))
    return Tensor(_handle=out)


def ones(shape, dtype: str = "float32") -> Tensor:
    out = _new(shape, dtype)
    _kernel("ones")(TensorIterator([], [out]))
    return Tensor(_handle=out)


def full(shape, value: float, dtype: str = "float32") -> Tensor:
    out = _new(shape, dtype)
    _kernel("full")(TensorIterator([], [out], {"fillValue": value}))
    return Tensor(_handle=out)


def empty(shape, dtype: str = "float32") -> Tensor:
    return Tensor(_handle=_new(shape, dtype))


def manualSeed(seed: int) -> None:
    """Seeds the generator behind `randn` (packages/types/src/random.ts:52-60)."""
    from .kernels import RandomState
    RandomState.manual_seed(seed)


def randn(shape, dtype: str = "float32") -> Tensor:
    """N(0,1) numbers from the device generator (packages/core/src/generated/internal/randn.ts)."""
    out = _new(shape, dtype)
    _kernel("randn")(TensorIterator([], [out]))
    return Tensor(_handle=out)


def arange(start, end=None, step=1, dtype: str = "int32") -> Tensor:
    if end is None:
        start, end = 0, start
    n = max(0, int(math.ceil((end - start) / step)))
    out = _new((n,), dtype)
    _kernel("arange")(TensorIterator([], [out], {"start": start, "step": step}))
    return Tensor(_handle=out)


def cat(tensors: Sequence[Tensor], dim: int = 0) -> Tensor:
    """Concatenation as slice-view + copy_ per input (one `copy` kernel call each)."""
    first = tensors[0]
    dim = dim % first.ndim
    total = sum(t.shape[dim] for t in tensors)
    shape = list(first.shape)
    shape[dim] = total
    dtype = first.dtype
    for t in tensors[1:]:
        dtype = _promote(dtype, t.dtype)
    out = Tensor(_handle=_new(shape, dtype))
    pos = 0
    for t in tensors:
        items = [slice(None)] * first.ndim
        items[dim] = slice(pos, pos + t.shape[dim])
        v = out.slice(items)
        copy_(v, t)
        v.dispose()
        pos += t.shape[dim]
    return out


def unsqueeze(a: Tensor, dim: int) -> Tensor:
    return a.unsqueeze(dim)


def expand(a: Tensor, shape) -> Tensor:
    return a.expand(shape)


def slice_(a: Tensor, spec) -> Tensor:
    return a.slice(spec)


def select(a: Tensor, dim: int, index: int) -> Tensor:
    return a.select(dim, index)


def argmax(a: Tensor, dim: int = -1, keepdim: bool = False) -> Tensor:
    """argmax over one dimension; logical int64 result (the WebGPU backend backs it with i32)."""
    dim = dim % a.ndim
    src = a
    moved = None
    if dim != a.ndim - 1:
        dims = [d for d in range(a.ndim) if d != dim] + [dim]
        moved = a.permute(dims)
        src = moved
    out_shape = src.shape[:-1]
    out = _new(out_shape, "int64")
    _kernel("argmax")(TensorIterator([src._handle], [out], {"dim": dim}))
    if moved is not None:
        moved.dispose()
    res = Tensor(_handle=out)
    if keepdim:
        r2 = res.unsqueeze(dim)
        res.dispose()
        return r2
    return res


# ----------------------------------------------------------------------------- matmul / linear
def matmul(a: Tensor, b: Tensor, *, transposeA: bool = False, transposeB: bool = False, alpha: float = 1.0,
           beta: float = 0.0, inputC: Tensor | None = None) -> Tensor:
    """`dispatchMatmul` (packages/core/src/dispatch/matmulOps.ts:408-496): shapes, batch broadcast
    and the MatmulDispatchResult handed to the backend's `matmul` kernel."""
    if a.ndim < 1 or b.ndim < 1:
        raise ValueError("matmul: both arguments must be at least 1-D")
    a_was_1d, b_was_1d = a.ndim == 1, b.ndim == 1
    av = a.unsqueeze(0) if a_was_1d else a
    bv = b.unsqueeze(1) if b_was_1d else b
    if av.ndim > 4 or bv.ndim > 4:
        raise ValueError("matmul: operands of rank > 4 are not supported")
    M, K = (av.shape[-1], av.shape[-2]) if transposeA else (av.shape[-2], av.shape[-1])
    K2, N = (bv.shape[-1], bv.shape[-2]) if transposeB else (bv.shape[-2], bv.shape[-1])
    if K != K2:
        raise ValueError(f"matmul: inner dimensions do not match ({K} vs {K2}); shapes {a.shape} @ {b.shape}")
    batch = _broadcast_shape(av.shape[:-2], bv.shape[:-2])
    out = _new(batch + (M, N), _promote(a.dtype, b.dtype))
    variant = "mm" if not batch else "bmm"
    cfg = MatmulDispatchResult(variant, out, M, K, N, batch, transposeA, transposeB, alpha, beta,
                               inputC._handle if inputC is not None else None)
    _kernel("matmul")(cfg, av._handle, bv._handle)
    if a_was_1d:
        av.dispose()
    if b_was_1d:
        bv.dispose()
    res = Tensor(_handle=out)
    if a_was_1d or b_was_1d:
        shape = list(res.shape)
        if b_was_1d:
            shape.pop(-1)
        if a_was_1d:
            shape.pop(-2 if not b_was_1d else -1)
        r2 = res.view(shape)
        res.dispose()
        return r2
    return res


def linear(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    """`linear` composite (packages/core/src/dispatch/handlers/composite.ts:55-77):
    matmul(x, weight, transposeB=true), then a separate broadcast `add` of the bias."""
    if x.shape[-1] != weight.shape[-1]:
        raise ValueError(f"linear: input features {x.shape[-1]} do not match weight {weight.shape}")
    xv, flat = x, None
    if x.ndim == 1:
        xv = x.unsqueeze(0)
    y = matmul(xv, weight, transposeB=True)
    if x.ndim == 1:
        xv.dispose()
        y2 = y.view((weight.shape[0],))
        y.dispose()
        y = y2
    if bias is not None:
        yb = add(y, bias)
        y.dispose()
        return yb
    return y


def embedding(ids: Tensor, weight: Tensor) -> Tensor:
    """`embedding` composite -> flatten ids (view) -> index_select(dim 0) -> view
    (packages/core/src/dispatch/handlers/composite.ts:149-245, handlers/gather.ts:97-137)."""
    if ids.dtype not in ("int32", "int64"):
        raise ValueError("embedding indices must be int32 or int64")
    flat = ids.reshape(-1)
    out = _new((flat.numel, weight.shape[1]), weight.dtype)
    _kernel("index_select")(weight._handle, flat._handle, {"dim": 0}, out)
    flat.dispose()
    res = Tensor(_handle=out)
    r2 = res.view(tuple(ids.shape) + (weight.shape[1],))
    res.dispose()
    return r2


# ----------------------------------------------------------------------------- normalize
def rmsNorm(x: Tensor, normalizedShape, weight: Tensor | None = None, eps: float = 1e-5) -> Tensor:
    if tuple(normalizedShape) != tuple(x.shape[-len(normalizedShape):]) or len(normalizedShape) != 1:
        raise ValueError("rms_norm: normalizedShape must equal the last dimension")
    h = _kernel("rms_norm")([x._handle], {"normalizedShape": tuple(normalizedShape), "eps": eps,
                                          "weight": weight._handle if weight is not None else None})
    return Tensor(_handle=h)


def layerNorm(x: Tensor, normalizedShape, weight: Tensor | None = None, bias: Tensor | None = None,
              eps: float = 1e-5) -> Tensor:
    if tuple(normalizedShape) != tuple(x.shape[-len(normalizedShape):]) or len(normalizedShape) != 1:
        raise ValueError("layer_norm: normalizedShape must equal the last dimension")
    h = _kernel("layer_norm")([x._handle], {"normalizedShape": tuple(normalizedShape), "eps": eps,
                                            "weight": weight._handle if weight is not None else None,
                                            "bias": bias._handle if bias is not None else None})
    return Tensor(_handle=h)


def softmax(x: Tensor, dim: int = -1) -> Tensor:
    dim = dim % x.ndim
    if dim != x.ndim - 1:
        raise ValueError("softmax: only the last dimension is supported")
    return Tensor(_handle=_kernel("softmax")([x._handle], {"dim": dim}))


# ----------------------------------------------------------------------------- attention
def scaledDotProductAttention(q: Tensor, k: Tensor, v: Tensor, attnMask: Tensor | None = None,
                              dropoutP: float = 0.0, isCausal: bool = False, scale: float | None = None) -> Tensor:
    """`scaled_dot_product_attention` composite
    (packages/core/src/dispatch/handlers/composite.ts:247-348): default scale 1/sqrt(E); with a
    mask the naive matmul(alpha=scale) -> add -> softmax -> matmul path; otherwise the backend's
    `flash_attention` kernel, falling back to the naive path when the backend lacks it."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if isCausal and attnMask is not None:
        raise ValueError("isCausal=true cannot be used with attnMask")
    fa = _backend().operators.find("flash_attention")
    if attnMask is None and fa is not None:
        out = _new(q.shape, q.dtype)
        fa(q._handle, k._handle, v._handle, out, float(scale), bool(isCausal))
        return Tensor(_handle=out)
    scores = matmul(q, k, transposeB=True, alpha=scale)
    mask = attnMask
    own_mask = False
    if mask is None and isCausal:
        sq, sk = q.shape[-2], k.shape[-2]
        m = np.where(np.arange(sk)[None, :] > np.arange(sq)[:, None], -np.inf, 0.0).astype(np.float32)
        mask, own_mask = Tensor(m, dtype="float32"), True
    if mask is not None:
        s2 = add(scores, mask)
        scores.dispose()
        scores = s2
        if own_mask:
            mask.dispose()
    probs = softmax(scores, -1)
    scores.dispose()
    out = matmul(probs, v)
    probs.dispose()
    return out


def conv1d(x: Tensor, weight: Tensor, bias: Tensor | None = None, stride: int = 1, padding: int = 0) -> Tensor:
    """conv1d through the window handler (packages/core/src/dispatch/handlers/window.ts:165-247)."""
    if x.ndim != 3 or weight.ndim != 3:
        raise ValueError("conv1d expects input [B,C,L] and weight [Cout,Cin,k]")
    if x.shape[1] != weight.shape[1]:
        raise ValueError(f"conv1d: input has {x.shape[1]} channels, weight expects {weight.shape[1]}")
    wout = (x.shape[2] + 2 * padding - weight.shape[2]) // stride + 1
    cfg = ConvDispatchResult(stride, padding, (x.shape[0], weight.shape[0], wout), _promote(x.dtype, weight.dtype))
    h = _kernel("conv1d")(cfg, x._handle, weight._handle, bias._handle if bias is not None else None)
    return Tensor(_handle=h)


class functional:
    """Namespace mirror of the reference's `functional` object (packages/core/src/generated/ops.ts)."""
    add = staticmethod(add)
    sub = staticmethod(sub)
    mul = staticmethod(mul)
    div = staticmethod(div)
    neg = staticmethod(neg)
    cos = staticmethod(cos)
    sin = staticmethod(sin)
    silu = staticmethod(silu)
    gelu = staticmethod(gelu)
    tanh = staticmethod(tanh)
    sigmoid = staticmethod(sigmoid)
    matmul = staticmethod(matmul)
    linear = staticmethod(linear)
    embedding = staticmethod(embedding)
    rmsNorm = staticmethod(rmsNorm)
    layerNorm = staticmethod(layerNorm)
    softmax = staticmethod(softmax)
    scaledDotProductAttention = staticmethod(scaledDotProductAttention)
    conv1d = staticmethod(conv1d)
    argmax = staticmethod(argmax)
