"""bf16 fast path of the Whisper audio encoder: the operator sequence of
`WhisperAudioEncoder.forward` (packages/model-utils/src/whisper/encoder.ts:202-250) with each
transformer block (packages/model-utils/src/whisper/block.ts:150-200 and
packages/core/src/nn/modules/attention/MultiheadAttention.ts:280-437) reduced to seven launches:

    LayerNorm -> packed QKV GEMM (+ in_proj_bias) -> flash attention on strided head views
    -> out_proj GEMM (+ bias + residual) -> LayerNorm -> fc1 GEMM (+ bias + GELU)
    -> fc2 GEMM (+ bias + residual)

The eager module projects q, k and v separately from row slices of `in_proj_weight` applied to
(L,N,E) views and copies every head layout; here the packed weight is used as it is stored
([3E,E], one GEMM), the result stays batch-first, and the attention kernel reads q/k/v through
strided [N,H,L,D] views of that one buffer and writes its output straight into [N,L,E].  Biases,
the tanh-form GELU and the residual adds run in the GEMM epilogue on the fp32 accumulator, so the
activations are rounded to bf16 once per GEMM instead of once per operator.

The convolution stem runs token-major: the mel input is transposed once to [N,L,nMels], each
conv1d is a vectorised im2col (three input rows side by side) plus a GEMM against the tap-major
weight with bias and GELU in the epilogue, and the second one also adds the position table, so its
output is the [N,T,E] stream the blocks work on (no channel-first intermediate, no transposes).
The final LayerNorm goes through the same operator kernel as the eager module.  The engine borrows
the parameters of a loaded `WhisperAudioEncoder` (only the two conv weights are re-laid out) and
needs bf16 storage; anything else raises.
"""
from __future__ import annotations

import ctypes
import math

from . import core, lib
from .core import Tensor
from .model_utils.whisper import WhisperAudioEncoder

KD_ACT_NONE, KD_ACT_GELU = 0, 1


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


class WhisperEncoderEngine:
    def __init__(self, encoder: WhisperAudioEncoder):
        cfg = encoder.config
        if cfg.dtype != "bfloat16":
            raise ValueError("WhisperEncoderEngine needs a bfloat16 encoder")
        self.enc = encoder
        self.E, self.H = cfg.nAudioState, cfg.nAudioHead
        self.D = self.E // self.H
        if self.D not in (64, 128) or self.E % 8:
            raise ValueError(f"head_dim {self.D} is not handled by the tensor-core attention kernel (64 or 128)")
        self.scale = 1.0 / math.sqrt(self.D)       # scaledDotProductAttention's default, composite.ts:272-275
        if cfg.nMels % 8:
            raise ValueError("the token-major stem needs a multiple of 8 mel bins")
        # conv weights [Cout, Cin, 3] -> [Cout, 3*Cin] with the tap index in front of the channel index
        self.w1 = self._tap_major(encoder.conv1.weight)
        self.w2 = self._tap_major(encoder.conv2.weight)
        self._pos = None                           # (B, T, tensor): the position table repeated per clip

    @staticmethod
    def _tap_major(w: Tensor) -> Tensor:
        p = w.permute([0, 2, 1])
        c = core.contiguous(p)
        out = c.view(w.shape[0], w.shape[1] * w.shape[2])   # keeps the storage alive
        p.dispose()
        c.dispose()
        return out

    def _positions(self, B: int, T: int) -> Tensor:
        """embed_positions[:T] repeated B times, [B,T,E]: the residual operand of the conv2 GEMM."""
        if self._pos is not None and self._pos[0] == B and self._pos[1] == T:
            return self._pos[2]
        if self._pos is not None:
            self._pos[2].dispose()
        pos = self.enc.embed_positions.weight.slice([slice(0, T), slice(None)])
        out = core.empty((B, T, self.E), "bfloat16")
        core.copy_(out, pos)                       # broadcast copy
        pos.dispose()
        self._pos = (B, T, out)
        return out

    # ------------------------------------------------------------------ one block
    def _block(self, blk, x: Tensor) -> Tensor:
        B, T, E = x.shape
        H, D = self.H, self.D
        e = lambda *shape: core.empty(shape, "bfloat16")  # noqa: E731
        mha = blk.self_attn
        y = blk.self_attn_layer_norm(x)
        qkv = e(B, T, 3 * E)
        lib.call("kd_linear_bf16_bias", _r(y), _r(mha.in_proj_weight), _r(mha.in_proj_bias), None, KD_ACT_NONE, _r(qkv))
        heads = qkv.view(B, T, 3 * H, D)
        views = []
        for j in range(3):
            s = heads.slice([slice(None), slice(None), slice(j * H, (j + 1) * H), slice(None)])
            views.append(s.permute([0, 2, 1, 3]))       # [B,H,T,D], strides (T*3E, D, 3E, 1)
            s.dispose()
        attn = e(B, T, E)
        a4 = attn.view(B, T, H, D)
        o = a4.permute([0, 2, 1, 3])
        lib.call("kd_flash_attention", _r(views[0]), _r(views[1]), _r(views[2]), _r(o), ctypes.c_float(self.scale), 0)
        x1 = e(B, T, E)
        lib.call("kd_linear_bf16_bias", _r(attn), _r(mha.out_proj.weight), _r(mha.out_proj.bias), _r(x), KD_ACT_NONE, _r(x1))
        y2 = blk.final_layer_norm(x1)
        h = e(B, T, blk.fc1.weight.shape[0])
        lib.call("kd_linear_bf16_bias", _r(y2), _r(blk.fc1.weight), _r(blk.fc1.bias), None, KD_ACT_GELU, _r(h))
        x2 = e(B, T, E)
        lib.call("kd_linear_bf16_bias", _r(h), _r(blk.fc2.weight), _r(blk.fc2.bias), _r(x1), KD_ACT_NONE, _r(x2))
        for t in (y, qkv, heads, *views, attn, a4, o, x1, y2, h):
            t.dispose()
        return x2

    # ------------------------------------------------------------------ forward
    def forward(self, mel: Tensor) -> Tensor:
        """mel [B, nMels, 2T] bf16 -> [B, T, E] bf16."""
        if mel.dtype != "bfloat16":
            raise ValueError("WhisperEncoderEngine.forward needs a bfloat16 mel tensor")
        enc = self.enc
        B, _, L = mel.shape
        E = self.E
        T = (L + 2 - 3) // 2 + 1                   # conv2: kernel 3, stride 2, padding 1
        if T > enc.config.nAudioCtx:
            raise ValueError(f"{T} frames exceed the encoder context of {enc.config.nAudioCtx}")
        mt = mel.permute([0, 2, 1])
        mel_t = core.contiguous(mt)                # [B, L, nMels]
        h1 = core.empty((B, L, E), "bfloat16")
        lib.call("kd_conv1d_tokens_bf16", _r(mel_t), _r(self.w1), _r(enc.conv1.bias), None, KD_ACT_GELU, 3, 1, 1, _r(h1))
        x = core.empty((B, T, E), "bfloat16")
        pos = self._positions(B, T)
        lib.call("kd_conv1d_tokens_bf16", _r(h1), _r(self.w2), _r(enc.conv2.bias), _r(pos), KD_ACT_GELU, 3, 2, 1, _r(x))
        for t in (mt, mel_t, h1):
            t.dispose()
        for blk in enc.layers:
            x2 = self._block(blk, x)
            x.dispose()
            x = x2
        out = enc.layer_norm(x)
        x.dispose()
        return out
