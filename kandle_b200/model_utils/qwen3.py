"""Qwen3 on the eager operator path: the modules issue, through `kandle_b200.core`, the same
sequence of backend kernel calls as the reference's TypeScript modules (about 41 per decoder
layer).  This is the "models run unchanged" path; the fused fast path lives in
`kandle_b200.engine`.

Reference files: packages/model-utils/src/rope.ts, kv-cache.ts, attention/gqa.ts, mlp/swiglu.ts,
qwen3/decoder_layer.ts, qwen3/model.ts, qwen3/for_causal_lm.ts.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from .. import core, nn
from ..core import Tensor


@dataclass
class Qwen3Config:
    """Qwen3ModelConfig (packages/model-utils/src/qwen3/model.ts:45-84); defaults are the 0.6B
    values used by the reference playground (playground-node/src/qwen3/utils.ts:19-33)."""
    vocabSize: int = 151936
    hiddenSize: int = 1024
    intermediateSize: int = 3072
    numHiddenLayers: int = 28
    numAttentionHeads: int = 16
    numKeyValueHeads: int = 8
    headDim: int = 128
    rmsNormEps: float = 1e-6
    ropeTheta: float = 1e6
    attentionBias: bool = False
    dtype: str = "float32"


class RotaryEmbedding:
    """packages/model-utils/src/rope.ts:120-272."""

    def __init__(self, dim: int, base: float = 10000.0, dtype: str = "float32"):
        self.dim, self.base, self.dtype = dim, base, dtype
        half = dim // 2
        # inv_freq in JS doubles, stored as float32 (rope.ts:159-171)
        vals = np.array([1.0 / math.pow(base, i / half) for i in range(half)], dtype=np.float32)
        self.invFreq = Tensor(vals, dtype="float32", shape=(half,))

    def getPositionIds(self, seqLen: int, startPos: int = 0) -> Tensor:
        return core.arange(startPos, startPos + seqLen, 1, "int32")

    def forward(self, positions: Tensor):
        """positions (seqLen,) int32 -> cos, sin of shape (seqLen, dim)  (rope.ts:192-261)."""
        if positions.ndim != 1:
            raise ValueError("RotaryEmbedding.forward: only 1-D position tensors are supported here")
        seq, half = positions.shape[0], self.dim // 2
        pos_e = positions.unsqueeze(-1)
        inv_e0 = self.invFreq.unsqueeze(0)
        inv_e = inv_e0.expand((seq, half))
        pos_f = pos_e.expand((seq, half))
        freqs = core.mul(pos_f, inv_e)              # int32 * float32 -> float32 on device
        emb = core.cat([freqs, freqs], -1)
        c, s = core.cos(emb), core.sin(emb)
        for t in (pos_e, inv_e0, inv_e, pos_f, freqs, emb):
            t.dispose()
        if self.dtype != "float32":
            c2, s2 = core.cast(c, self.dtype), core.cast(s, self.dtype)
            c.dispose()
            s.dispose()
            c, s = c2, s2
        return {"cos": c, "sin": s}


def applyRotaryPosEmbDirect(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor, unsqueezeDim: int = 1):
    """packages/model-utils/src/rope.ts:546-644: x*cos + rotate_half(x)*sin, with
    rotate_half(x) = cat(-x[half:], x[:half]); per tensor: 2 slices (views), 2 contiguous, neg,
    cat (2 copies), 2 mul, add."""
    head_dim = q.shape[-1]
    if cos.shape[-1] != head_dim:
        raise ValueError(f"cos/sin last dimension ({cos.shape[-1]}) must equal head_dim ({head_dim}).")
    inter = []
    if cos.ndim == 2:
        c1, s1 = cos.unsqueeze(0), sin.unsqueeze(0)
        cos_e, sin_e = c1.unsqueeze(0), s1.unsqueeze(0)
        inter += [c1, s1, cos_e, sin_e]
    else:
        cos_e, sin_e = cos.unsqueeze(unsqueezeDim), sin.unsqueeze(unsqueezeDim)
        inter += [cos_e, sin_e]

    def rotate_half(x: Tensor):
        half = x.shape[-1] // 2
        a, b = x.slice(f"..., :{half}"), x.slice(f"..., {half}:")
        x1, x2 = core.contiguous(a), core.contiguous(b)
        n2 = core.neg(x2)
        res = core.cat([n2, x1], -1)
        for t in (a, b, x1, x2, n2):
            t.dispose()
        return res

    outs = []
    for x in (q, k):
        rot = rotate_half(x)
        xc = core.mul(x, cos_e)
        rs = core.mul(rot, sin_e)
        outs.append(core.add(xc, rs))
        for t in (rot, xc, rs):
            t.dispose()
    for t in inter:
        t.dispose()
    return outs[0], outs[1]


class StaticKVCache:
    """packages/model-utils/src/kv-cache.ts:92-309: zeros [B,Hkv,maxS,D] per layer, `update`
    = slice view + copy_ and returns [:, :, :end, :] views."""

    def __init__(self, numLayers: int, numKvHeads: int, headDim: int, maxSeqLen: int, batchSize: int = 1,
                 dtype: str = "float32"):
        self.numLayers, self.maxSeqLen, self.batchSize = numLayers, maxSeqLen, batchSize
        shape = (batchSize, numKvHeads, maxSeqLen, headDim)
        self.layers = [{"keyCache": core.zeros(shape, dtype), "valueCache": core.zeros(shape, dtype)}
                       for _ in range(numLayers)]
        self._seenTokens = 0

    def getLayerCache(self, layerIdx: int):
        if not 0 <= layerIdx < self.numLayers:
            raise IndexError(f"Layer index {layerIdx} out of range")
        return self.layers[layerIdx]

    def update(self, layerIdx: int, key: Tensor, value: Tensor, startPos: int):
        cache = self.getLayerCache(layerIdx)
        end = startPos + key.shape[2]
        if end > self.maxSeqLen:
            raise ValueError(f"Cache overflow: trying to write to position {startPos}-{end}, "
                             f"but maxSeqLen is {self.maxSeqLen}")
        spec = f":, :, {startPos}:{end}, :"
        for name, new in (("keyCache", key), ("valueCache", value)):
            v = cache[name].slice(spec)
            core.copy_(v, new)
            v.dispose()
        self._seenTokens = max(self._seenTokens, end)
        return cache["keyCache"].slice(f":, :, :{end}, :"), cache["valueCache"].slice(f":, :, :{end}, :")

    def getSeqLength(self) -> int:
        return self._seenTokens

    def rollback(self, toPos: int) -> None:
        self._seenTokens = min(self._seenTokens, toPos)

    def dispose(self) -> None:
        for l in self.layers:
            l["keyCache"].dispose()
            l["valueCache"].dispose()


class GroupedQueryAttention(nn.Module):
    """packages/model-utils/src/attention/gqa.ts:246-430 (flash path; `captureAttentionWeights`
    is not mirrored)."""

    def __init__(self, embedDim: int, numHeads: int, numKvHeads: int, headDim: int, bias: bool = False,
                 useQkNorm: bool = True, rmsNormEps: float = 1e-6, dtype: str = "float32"):
        super().__init__()
        self.numHeads, self.numKvHeads, self.headDim = numHeads, numKvHeads, headDim
        self.numKvGroups = numHeads // numKvHeads
        self.q_proj = nn.Linear(embedDim, numHeads * headDim, bias, dtype)
        self.k_proj = nn.Linear(embedDim, numKvHeads * headDim, bias, dtype)
        self.v_proj = nn.Linear(embedDim, numKvHeads * headDim, bias, dtype)
        self.o_proj = nn.Linear(numHeads * headDim, embedDim, bias, dtype)
        self.useQkNorm = useQkNorm
        if useQkNorm:
            self.q_norm = nn.RMSNorm(headDim, rmsNormEps, dtype)
            self.k_norm = nn.RMSNorm(headDim, rmsNormEps, dtype)

    def _permuteToHeadsFirst(self, x: Tensor) -> Tensor:      # gqa.ts:452-460
        p = x.permute([0, 2, 1, 3])
        c = core.contiguous(p)
        p.dispose()
        return c

    def _repeatKv(self, x: Tensor, bsz: int, kvLen: int) -> Tensor:   # gqa.ts:494-519
        u = x.unsqueeze(2)
        e = u.expand((bsz, self.numKvHeads, self.numKvGroups, kvLen, self.headDim))
        c = core.contiguous(e)
        r = c.view(bsz, self.numHeads, kvLen, self.headDim)
        for t in (u, e, c):
            t.dispose()
        return r

    def forward(self, hiddenStates: Tensor, *, isCausal: bool = False, positionEmbeddings=None,
                kvCacheUpdateFn=None, cachePosition: int = 0) -> Tensor:
        bsz, seqLen = hiddenStates.shape[0], hiddenStates.shape[1]
        qp, kp, vp = self.q_proj(hiddenStates), self.k_proj(hiddenStates), self.v_proj(hiddenStates)
        q = qp.view(bsz, seqLen, self.numHeads, self.headDim)
        k = kp.view(bsz, seqLen, self.numKvHeads, self.headDim)
        v = vp.view(bsz, seqLen, self.numKvHeads, self.headDim)
        if self.useQkNorm:
            qn, kn = self.q_norm(q), self.k_norm(k)
            q.dispose()
            k.dispose()
            q, k = qn, kn
        for t in (qp, kp, vp):
            t.dispose()
        qh, kh, vh = self._permuteToHeadsFirst(q), self._permuteToHeadsFirst(k), self._permuteToHeadsFirst(v)
        for t in (q, k, v):
            t.dispose()
        q, k, v = qh, kh, vh
        if positionEmbeddings is not None:
            q2, k2 = applyRotaryPosEmbDirect(q, k, positionEmbeddings["cos"], positionEmbeddings["sin"])
            q.dispose()
            k.dispose()
            q, k = q2, k2
        cachedK, cachedV, kvSeqLen = k, v, seqLen
        if kvCacheUpdateFn is not None:
            cachedK, cachedV = kvCacheUpdateFn(k, v, cachePosition)
            kvSeqLen = cachedK.shape[2]
        expK, expV = cachedK, cachedV
        if self.numKvGroups > 1:
            expK, expV = self._repeatKv(cachedK, bsz, kvSeqLen), self._repeatKv(cachedV, bsz, kvSeqLen)
        causal = isCausal
        if kvCacheUpdateFn is not None and seqLen == 1 and kvSeqLen > 1:
            causal = False                                         # gqa.ts:333-336
        attn = core.scaledDotProductAttention(q, expK, expV, None, 0.0, causal)
        m1 = attn.permute([0, 2, 1, 3])                            # gqa.ts:466-480
        m2 = core.contiguous(m1)
        merged = m2.view(bsz, seqLen, self.numHeads * self.headDim)
        out = self.o_proj(merged)
        seen = set()
        for t in (merged, m2, m1, attn, expK, expV, cachedK, cachedV, q, k, v):
            if id(t) not in seen:
                seen.add(id(t))
                t.dispose()
        return out


class SwiGLUMLP(nn.Module):
    """packages/model-utils/src/mlp/swiglu.ts:119-134: down(silu(gate(x)) * up(x))."""

    def __init__(self, hiddenSize: int, intermediateSize: int, dtype: str = "float32"):
        super().__init__()
        self.gate_proj = nn.Linear(hiddenSize, intermediateSize, False, dtype)
        self.up_proj = nn.Linear(hiddenSize, intermediateSize, False, dtype)
        self.down_proj = nn.Linear(intermediateSize, hiddenSize, False, dtype)

    def forward(self, x: Tensor) -> Tensor:
        g = self.gate_proj(x)
        a = core.silu(g)
        u = self.up_proj(x)
        h = core.mul(a, u)
        out = self.down_proj(h)
        for t in (g, a, u, h):
            t.dispose()
        return out


class Qwen3DecoderLayer(nn.Module):
    """packages/model-utils/src/qwen3/decoder_layer.ts:191-241 (pre-norm residual block)."""

    def __init__(self, cfg: Qwen3Config, layerIdx: int):
        super().__init__()
        self.layerIdx = layerIdx
        self.self_attn = GroupedQueryAttention(cfg.hiddenSize, cfg.numAttentionHeads, cfg.numKeyValueHeads,
                                               cfg.headDim, cfg.attentionBias, True, cfg.rmsNormEps, cfg.dtype)
        self.mlp = SwiGLUMLP(cfg.hiddenSize, cfg.intermediateSize, cfg.dtype)
        self.input_layernorm = nn.RMSNorm(cfg.hiddenSize, cfg.rmsNormEps, cfg.dtype)
        self.post_attention_layernorm = nn.RMSNorm(cfg.hiddenSize, cfg.rmsNormEps, cfg.dtype)

    def forward(self, h: Tensor, *, positionEmbeddings, kvCache: StaticKVCache | None = None,
                cachePosition: int = 0) -> Tensor:
        x = self.input_layernorm(h)
        upd = None
        if kvCache is not None:
            upd = lambda k, v, pos: kvCache.update(self.layerIdx, k, v, pos)  # noqa: E731
        a = self.self_attn(x, isCausal=True, positionEmbeddings=positionEmbeddings, kvCacheUpdateFn=upd,
                           cachePosition=cachePosition)
        h1 = core.add(h, a)
        x2 = self.post_attention_layernorm(h1)
        m = self.mlp(x2)
        h2 = core.add(h1, m)
        for t in (x, a, h1, x2, m):
            t.dispose()
        return h2


class Qwen3Model(nn.Module):
    """packages/model-utils/src/qwen3/model.ts:265-347."""

    def __init__(self, cfg: Qwen3Config):
        super().__init__()
        self.config = cfg
        self.embed_tokens = nn.Embedding(cfg.vocabSize, cfg.hiddenSize, cfg.dtype)
        self.layers = nn.ModuleList([Qwen3DecoderLayer(cfg, i) for i in range(cfg.numHiddenLayers)])
        self.norm = nn.RMSNorm(cfg.hiddenSize, cfg.rmsNormEps, cfg.dtype)
        self.rotary_emb = RotaryEmbedding(cfg.headDim, cfg.ropeTheta, cfg.dtype)

    def forward(self, inputIds: Tensor, kvCache: StaticKVCache | None = None, cachePosition: int = 0) -> Tensor:
        seqLen = inputIds.shape[1]
        h = self.embed_tokens(inputIds)
        pos = self.rotary_emb.getPositionIds(seqLen, cachePosition)
        pe = self.rotary_emb.forward(pos)
        pos.dispose()
        for layer in self.layers:
            h2 = layer(h, positionEmbeddings=pe, kvCache=kvCache, cachePosition=cachePosition)
            h.dispose()
            h = h2
        pe["cos"].dispose()
        pe["sin"].dispose()
        out = self.norm(h)
        h.dispose()
        return out


class Qwen3ForCausalLM(nn.Module):
    """packages/model-utils/src/qwen3/for_causal_lm.ts:107-194: tied lm_head computed as
    matmul(h, transpose(embed, 0, 1)) for every position."""

    def __init__(self, cfg: Qwen3Config):
        super().__init__()
        self.config = cfg
        self.model = Qwen3Model(cfg)

    def createKVCache(self, maxSeqLen: int, batchSize: int = 1, dtype: str | None = None) -> StaticKVCache:
        c = self.config
        return StaticKVCache(c.numHiddenLayers, c.numKeyValueHeads, c.headDim, maxSeqLen, batchSize, dtype or c.dtype)

    def _lm_head(self, h: Tensor) -> Tensor:
        wt = self.model.embed_tokens.weight.transpose(0, 1)       # strided [H,V] view
        logits = core.matmul(h, wt)
        wt.dispose()
        return logits

    def forward(self, inputIds: Tensor) -> Tensor:
        h = self.model(inputIds)
        logits = self._lm_head(h)
        h.dispose()
        return logits

    def forwardWithKVCache(self, inputIds: Tensor, kvCache: StaticKVCache, cachePosition: int) -> Tensor:
        h = self.model(inputIds, kvCache, cachePosition)
        logits = self._lm_head(h)
        h.dispose()
        return logits

    def generateGreedy(self, inputIds: Tensor, steps: int, maxSeqLen: int | None = None) -> np.ndarray:
        """Batch-capable greedy loop built from the public pieces (forwardWithKVCache, select of
        the last position, argmax), the batched form of generateWithKVCache
        (for_causal_lm.ts:475-508).  Returns int64 [B, steps]."""
        B, S = inputIds.shape
        cache = self.createKVCache(maxSeqLen or S + steps, B)
        out = np.empty((B, steps), dtype=np.int64)
        ids, pos = inputIds, 0
        for t in range(steps):
            logits = self.forwardWithKVCache(ids, cache, pos)
            last = logits.select(1, logits.shape[1] - 1)
            tok = core.argmax(last, 1)
            out[:, t] = tok.dataAsync()
            pos += ids.shape[1]
            if ids is not inputIds:
                ids.dispose()
            nxt = tok.view(B, 1)
            ids = core.cast(nxt, "int32")
            for x in (logits, last, tok, nxt):
                x.dispose()
        if ids is not inputIds:
            ids.dispose()
        cache.dispose()
        return out
