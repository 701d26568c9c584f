"""Whisper audio encoder on the eager operator path.

Reference files: packages/model-utils/src/whisper/config.ts:33-69, whisper/encoder.ts:202-250,
whisper/block.ts:150-200, packages/core/src/nn/modules/attention/MultiheadAttention.ts:280-437.
`embed_positions.weight` is a plain parameter: the reference module never initialises it
(encoder.ts:175-180), so the caller loads it with the rest of the state dict.
"""
from __future__ import annotations

from dataclasses import dataclass

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


class ResidualAttentionBlock(nn.Module):
    """Pre-LN self-attention + GELU MLP block (whisper/block.ts:150-200)."""

    def __init__(self, cfg: WhisperConfig):
        super().__init__()
        E = cfg.nAudioState
        self.self_attn_layer_norm = nn.LayerNorm(E, cfg.layerNormEps, cfg.dtype)
        self.self_attn = nn.MultiheadAttention(E, cfg.nAudioHead, cfg.dtype)
        self.final_layer_norm = nn.LayerNorm(E, cfg.layerNormEps, cfg.dtype)
        self.fc1 = nn.Linear(E, 4 * E, True, cfg.dtype)
        self.fc2 = nn.Linear(4 * E, E, True, cfg.dtype)

    def forward(self, x: Tensor) -> Tensor:
        y = self.self_attn_layer_norm(x)
        a = self.self_attn(y)
        x1 = core.add(x, a)                 # strided rhs (batch-first view of an (L,N,E) tensor)
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
