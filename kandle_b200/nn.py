"""Mirror of the `nn` modules the Qwen3 and Whisper models are built from
(packages/core/src/nn): Module, Linear, Embedding, RMSNorm, LayerNorm, Conv1d, GELU,
MultiheadAttention.  Parameters are `Tensor`s created zero-initialised and filled through
`loadStateDict` (the reference loads safetensors through the same path, nn/module.ts:462-669).
`call()` is synchronous here; in the reference it is `async` only to await hooks.
"""
from __future__ import annotations

import numpy as np

from . import core
from .core import Tensor


class Module:
    """packages/core/src/nn/module.ts:106."""

    def __init__(self):
        object.__setattr__(self, "_parameters", {})
        object.__setattr__(self, "_modules", {})

    def __setattr__(self, name, value):
        if isinstance(value, Tensor):
            self._parameters[name] = value
        elif isinstance(value, Module):
            self._modules[name] = value
        object.__setattr__(self, name, value)

    def registerParameter(self, name: str, t: Tensor | None) -> None:
        setattr(self, name, t)

    def registerBuffer(self, name: str, t: Tensor, persistent: bool = True) -> None:
        """nn/module.ts registerBuffer: a non-persistent buffer is an attribute that stays out of the state dict."""
        if persistent:
            setattr(self, name, t)
        else:
            object.__setattr__(self, name, t)

    def namedParameters(self, prefix: str = ""):
        for n, p in self._parameters.items():
            yield prefix + n, p
        for mn, m in self._modules.items():
            yield from m.namedParameters(prefix + mn + ".")

    def stateDict(self) -> dict:
        return dict(self.namedParameters())

    def loadStateDict(self, state: dict, strict: bool = True) -> None:
        """Copies host arrays into the parameters (shape-checked), nn/module.ts:501."""
        be = core._backend()
        own = self.stateDict()
        missing = [k for k in own if k not in state]
        if strict and missing:
            raise KeyError(f"missing keys in state dict: {missing[:5]}{'...' if len(missing) > 5 else ''}")
        for k, p in own.items():
            if k not in state:
                continue
            arr = np.asarray(state[k])
            if tuple(arr.shape) != tuple(p.shape):
                raise ValueError(f"shape mismatch for {k}: {arr.shape} vs {p.shape}")
            be.upload(p._handle, arr)

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def call(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    __call__ = call


class ModuleList(Module):
    def __init__(self, modules=()):
        super().__init__()
        self._list = []
        for m in modules:
            self.append(m)

    def append(self, m: Module) -> None:
        self._modules[str(len(self._list))] = m
        self._list.append(m)

    def __iter__(self):
        return iter(self._list)

    def __len__(self):
        return len(self._list)

    def __getitem__(self, i):
        return self._list[i]


class Linear(Module):
    """packages/core/src/nn/modules/linear; weight [out,in], y = x W^T + b."""

    def __init__(self, inFeatures: int, outFeatures: int, bias: bool = True, dtype: str = "float32"):
        super().__init__()
        self.inFeatures, self.outFeatures = inFeatures, outFeatures
        self.weight = core.zeros((outFeatures, inFeatures), dtype)
        self.bias = core.zeros((outFeatures,), dtype) if bias else None

    def forward(self, x: Tensor) -> Tensor:
        return core.linear(x, self.weight, self.bias)


class Embedding(Module):
    def __init__(self, numEmbeddings: int, embeddingDim: int, dtype: str = "float32"):
        super().__init__()
        self.numEmbeddings, self.embeddingDim = numEmbeddings, embeddingDim
        self.weight = core.zeros((numEmbeddings, embeddingDim), dtype)

    def forward(self, ids: Tensor) -> Tensor:
        return core.embedding(ids, self.weight)


class RMSNorm(Module):
    """packages/core/src/nn/modules/normalization/RMSNorm.ts:40-99 (weight initialised to ones,
    eps default 1e-6 at module level)."""

    def __init__(self, normalizedShape, eps: float = 1e-6, dtype: str = "float32"):
        super().__init__()
        self.normalizedShape = (normalizedShape,) if isinstance(normalizedShape, int) else tuple(normalizedShape)
        self.eps = eps
        self.weight = core.ones(self.normalizedShape, dtype)

    def forward(self, x: Tensor) -> Tensor:
        return core.rmsNorm(x, self.normalizedShape, self.weight, self.eps)


class LayerNorm(Module):
    def __init__(self, normalizedShape, eps: float = 1e-5, dtype: str = "float32"):
        super().__init__()
        self.normalizedShape = (normalizedShape,) if isinstance(normalizedShape, int) else tuple(normalizedShape)
        self.eps = eps
        self.weight = core.ones(self.normalizedShape, dtype)
        self.bias = core.zeros(self.normalizedShape, dtype)

    def forward(self, x: Tensor) -> Tensor:
        return core.layerNorm(x, self.normalizedShape, self.weight, self.bias, self.eps)


class GELU(Module):
    def forward(self, x: Tensor) -> Tensor:
        return core.gelu(x)


class Conv1d(Module):
    def __init__(self, inChannels: int, outChannels: int, kernelSize: int, stride: int = 1, padding: int = 0,
                 bias: bool = True, dtype: str = "float32"):
        super().__init__()
        self.stride, self.padding = stride, padding
        self.weight = core.zeros((outChannels, inChannels, kernelSize), dtype)
        self.bias = core.zeros((outChannels,), dtype) if bias else None

    def forward(self, x: Tensor) -> Tensor:
        return core.conv1d(x, self.weight, self.bias, self.stride, self.padding)


class MultiheadAttention(Module):
    """packages/core/src/nn/modules/attention/MultiheadAttention.ts:280-437 (batchFirst=true), self- and
    cross-attention: inputs are transposed to (L,N,E) views, q/k/v projections use row slices of
    `in_proj_weight` / `in_proj_bias` (views with non-zero offsets), heads become (N*H, L, E/H) and
    attention runs through scaledDotProductAttention on 3-D tensors."""

    def __init__(self, embedDim: int, numHeads: int, dtype: str = "float32"):
        super().__init__()
        self.embedDim, self.numHeads, self.headDim = embedDim, numHeads, embedDim // numHeads
        self.in_proj_weight = core.zeros((3 * embedDim, embedDim), dtype)
        self.in_proj_bias = core.zeros((3 * embedDim,), dtype)
        self.out_proj = Linear(embedDim, embedDim, True, dtype)

    def forward(self, query: Tensor, key: Tensor | None = None, value: Tensor | None = None,
                attnMask: Tensor | None = None) -> Tensor:
        """query (N,L,E); key/value (N,S,E), default: the query (self-attention).  attnMask is an
        additive float mask broadcastable to (N*H, L, S); with a mask scaledDotProductAttention takes
        the naive matmul -> add -> softmax -> matmul path, as the reference does."""
        E, H, D = self.embedDim, self.numHeads, self.headDim
        srcs = [query, query if key is None else key, query if value is None else value]
        N = query.shape[0]
        outs = []
        for j in range(3):
            x = srcs[j].transpose(0, 1)                # (L or S, N, E) view
            Lj = x.shape[0]
            w = self.in_proj_weight.slice([slice(j * E, (j + 1) * E), slice(None)])
            b = self.in_proj_bias.slice([slice(j * E, (j + 1) * E)])
            p = core.linear(x, w, b)                   # (Lj, N, E)
            w.dispose()
            b.dispose()
            v1 = p.view(Lj, N * H, D)
            v2 = v1.permute([1, 0, 2])                 # (N*H, Lj, D)
            outs.append(core.contiguous(v2))
            for t in (v2, v1, p, x):
                t.dispose()
        L = query.shape[1]
        q, k, v = outs
        o = core.scaledDotProductAttention(q, k, v, attnMask, 0.0, False)
        for t in outs:
            t.dispose()
        o1 = o.permute([1, 0, 2])                      # (L, N*H, D)
        o2 = core.contiguous(o1)
        o3 = o2.view(L, N, E)
        y = self.out_proj(o3)                          # (L, N, E)
        for t in (o3, o2, o1, o):
            t.dispose()
        yt = y.transpose(0, 1)                         # back to batch-first, non-contiguous view
        y.dispose()
        return yt
