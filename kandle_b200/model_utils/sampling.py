"""Mirror of `@kandle/model-utils` sampling (packages/model-utils/src/sampling/index.ts): `sample`
and `sampleGreedy` with the reference's SamplerConfig / SampleResult names, computed on the device
by kd_sample instead of a host sort of the downloaded logits."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import numpy as np

from .. import core, lib
from ..core import Tensor


@dataclass
class SamplerConfig:                      # index.ts:23-55, defaults :77-82
    temperature: float = 1.0
    topK: int = 0
    topP: float = 1.0
    doSample: bool = True


@dataclass
class SampleResult:                       # index.ts:60-72
    tokenId: int
    logProb: float
    topKTokenIds: list = field(default_factory=list)
    topKProbs: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


def sample(logits: Tensor, config: SamplerConfig | None = None, displayTopK: int = 0, uniform: float | None = None,
           rng: np.random.Generator | None = None) -> SampleResult:
    """logits [V] or [1, V] fp32 on the device.  The draw uses `uniform` in [0, 1) if given, else one
    number from `rng` (default: numpy's global generator) where the reference calls Math.random().
    displayTopK > 0 additionally downloads the row to build the reference's display list of the
    largest logits with their probabilities under the plain softmax at `temperature` (the greedy
    branch's list, index.ts:142-153); leave it at 0 on the token path."""
    cfg = config or SamplerConfig()
    if logits.dtype != "float32":
        raise TypeError("sample expects float32 logits")
    if len(logits.shape) == 2 and logits.shape[0] != 1:
        raise ValueError("sample takes one row of logits: [V] or [1, V]")
    ids = core.zeros((1,), "int64")
    lp = core.zeros((1,), "float32")
    u = None
    if cfg.doSample:
        r = uniform if uniform is not None else (rng.random() if rng is not None else np.random.random())
        u = Tensor(np.array([r], dtype=np.float32))
    lib.call("kd_sample", _r(logits), ctypes.c_double(cfg.temperature), int(cfg.topK), ctypes.c_double(cfg.topP),
             1 if cfg.doSample else 0, _r(u), _r(ids), _r(lp))
    res = SampleResult(int(ids.dataAsync()[0]), float(lp.dataAsync()[0]))
    if displayTopK > 0:
        row = logits.dataAsync().reshape(-1).astype(np.float64)
        order = np.argsort(-row, kind="stable")[:displayTopK]
        e = np.exp((row - row.max()) / cfg.temperature)
        res.topKTokenIds = [int(i) for i in order]
        res.topKProbs = (e[order] / e.sum()).astype(np.float32)
    return res


def sampleGreedy(logits: Tensor, displayTopK: int = 0) -> SampleResult:    # index.ts:243-248
    return sample(logits, SamplerConfig(doSample=False), displayTopK)
