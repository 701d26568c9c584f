"""Whisper audio encoder and text decoder on the eager operator path.

Reference files: packages/model-utils/src/whisper/config.ts:33-69, whisper/encoder.ts:202-250,
whisper/block.ts:150-200, packages/core/src/nn/modules/attention/MultiheadAttention.ts:280-437.
Decoder: whisper/decoder.ts:82-262 (token + learned position embeddings, blocks with causal
self-attention through an additive -inf mask and cross-attention over the encoder output, final
LayerNorm, logits through the transposed token embedding).
`embed_positions.weight` is a plain parameter: the reference module never initialises it
(encoder.ts:175-180), so the caller loads it with the rest of the state dict.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .. import core, nn
from ..core import Tensor


@dataclass
class WhisperConfig:
    nMels: int = 80
    nAudioCtx: int = 1500
    nAudioState: int = 768
    nAudioHead: int = 12
    nAudioLayer: int = 12
    layerNormEps: float = 1e-5
    dtype: str = "float32"
    # text decoder (config.ts: vocabSize, maxTargetPositions, dModel, decoderAttentionHeads, decoderLayers)
    nVocab: int = 51865
    nTextCtx: int = 448
    nTextState: int = 768
    nTextHead: int = 12
    nTextLayer: int = 12


class ResidualAttentionBlock(nn.Module):
    """Pre-LN self-attention (+ optional cross-attention) + GELU MLP block (whisper/block.ts:150-200)."""

    def __init__(self, cfg: WhisperConfig, crossAttention: bool = False, nState: int | None = None, nHead: int | None = None):
        super().__init__()
        E = nState or cfg.nAudioState
        H = nHead or cfg.nAudioHead
        self.self_attn_layer_norm = nn.LayerNorm(E, cfg.layerNormEps, cfg.dtype)
        self.self_attn = nn.MultiheadAttention(E, H, cfg.dtype)
        self.encoder_attn = None
        if crossAttention:
            self.encoder_attn_layer_norm = nn.LayerNorm(E, cfg.layerNormEps, cfg.dtype)
            self.encoder_attn = nn.MultiheadAttention(E, H, cfg.dtype)
        self.final_layer_norm = nn.LayerNorm(E, cfg.layerNormEps, cfg.dtype)
        self.fc1 = nn.Linear(E, 4 * E, True, cfg.dtype)
        self.fc2 = nn.Linear(4 * E, E, True, cfg.dtype)

    def forward(self, x: Tensor, xa: Tensor | None = None, mask: Tensor | None = None) -> Tensor:
        y = self.self_attn_layer_norm(x)
        a = self.self_attn(y, None, None, mask)
        x1 = core.add(x, a)                 # strided rhs (batch-first view of an (L,N,E) tensor)
        if self.encoder_attn is not None and xa is not None:
            yc = self.encoder_attn_layer_norm(x1)
            ac = self.encoder_attn(yc, xa, xa)
            xc = core.add(x1, ac)
            for t in (yc, ac, x1):
                t.dispose()
            x1 = xc
        y2 = self.final_layer_norm(x1)
        h = self.fc1(y2)
        g = core.gelu(h)
        m = self.fc2(g)
        x2 = core.add(x1, m)
        for t in (y, a, x1, y2, h, g, m):
            t.dispose()
        return x2


class WhisperAudioEncoder(nn.Module):
    """whisper/encoder.ts:202-250: conv1 -> gelu -> conv2 (stride 2) -> gelu -> permute(0,2,1) ->
    + embed_positions[:T] -> blocks -> layer_norm."""

    def __init__(self, cfg: WhisperConfig):
        super().__init__()
        self.config = cfg
        E = cfg.nAudioState
        self.conv1 = nn.Conv1d(cfg.nMels, E, 3, 1, 1, True, cfg.dtype)
        self.conv2 = nn.Conv1d(E, E, 3, 2, 1, True, cfg.dtype)
        self.embed_positions = nn.Embedding(cfg.nAudioCtx, E, cfg.dtype)
        self.layers = nn.ModuleList([ResidualAttentionBlock(cfg) for _ in range(cfg.nAudioLayer)])
        self.layer_norm = nn.LayerNorm(E, cfg.layerNormEps, cfg.dtype)

    def forward(self, mel: Tensor) -> Tensor:
        c1 = self.conv1(mel)
        g1 = core.gelu(c1)
        c2 = self.conv2(g1)
        g2 = core.gelu(c2)
        xt = g2.permute([0, 2, 1])                      # [B,T,C], non-contiguous view
        T = xt.shape[1]
        pos = self.embed_positions.weight.slice([slice(0, T), slice(None)])
        x = core.add(xt, pos)
        for t in (c1, g1, c2, g2, xt, pos):
            t.dispose()
        for blk in self.layers:
            x2 = blk(x)
            x.dispose()
            x = x2
        out = self.layer_norm(x)
        x.dispose()
        return out


class WhisperTextDecoder(nn.Module):
    """whisper/decoder.ts:82-262: embed_tokens(tokens) + embed_positions[offset:offset+S] -> blocks with
    (x, xa, mask[:S,:S]) -> layer_norm -> matmul with embed_tokens.weight transposed."""

    def __init__(self, cfg: WhisperConfig):
        super().__init__()
        self.config = cfg
        E = cfg.nTextState
        self.embed_tokens = nn.Embedding(cfg.nVocab, E, cfg.dtype)
        self.embed_positions = nn.Embedding(cfg.nTextCtx, E, cfg.dtype)
        self.layers = nn.ModuleList([ResidualAttentionBlock(cfg, True, E, cfg.nTextHead) for _ in range(cfg.nTextLayer)])
        self.layer_norm = nn.LayerNorm(E, cfg.layerNormEps, cfg.dtype)
        n = cfg.nTextCtx
        m = np.where(np.arange(n)[None, :] > np.arange(n)[:, None], -np.inf, 0.0).astype(np.float32)   # decoder.ts:153-165
        self.registerBuffer("mask", Tensor(m, dtype=cfg.dtype), False)     # decoder.ts:166: not persisted

    def forward(self, tokens: Tensor, xa: Tensor, offset: int = 0) -> Tensor:
        S = tokens.shape[1]
        if offset + S > self.config.nTextCtx:
            raise ValueError(f"positions {offset}..{offset + S} exceed the decoder context of {self.config.nTextCtx}")
        e = self.embed_tokens(tokens)
        pos = self.embed_positions.weight.slice([slice(offset, offset + S), slice(None)])
        x = core.add(e, pos)
        mask = self.mask.slice([slice(0, S), slice(0, S)])
        for t in (e, pos):
            t.dispose()
        for blk in self.layers:
            x2 = blk(x, xa, mask)
            x.dispose()
            x = x2
        y = self.layer_norm(x)
        wt = self.embed_tokens.weight.transpose(0, 1)
        logits = core.matmul(y, wt)
        for t in (x, y, wt, mask):
            t.dispose()
        return logits
