"""bf16 fast path of the Whisper text decoder with a self-attention KV cache and the encoder's
keys / values projected once per clip.

The reference's decoder forward (packages/model-utils/src/whisper/decoder.ts:203-261, blocks
whisper/block.ts:150-200, packages/core/src/nn/modules/attention/MultiheadAttention.ts:280-437)
recomputes every position of the text and re-projects the 1500 encoder frames in every layer at
every step.  Here a step costs what it must:

    set_audio(xa)     per layer ONE GEMM: xa x in_proj_weight[E:3E]^T (+ bias) -> packed K|V of the clip,
                      kept; the attention kernels read K and V as strided [B,H,S,D] views of it
    forward(tokens)   the prompt (positions 0..T-1): packed QKV GEMM, K/V rows into the cache, causal
                      flash attention, cross attention on the cached K|V, bias / GELU / residual in
                      the GEMM epilogues
    step(tokens)      one new position per clip: the same with the split-KV decode attention kernel
                      (one query per sequence against the cache prefix, and against the 1500 frames)

Numerics as the encoder fast path: bf16 operands, fp32 accumulation, one rounding per GEMM.  The
additive -inf mask of the reference's self-attention equals the causal mask of the fused kernel
(whisper/decoder.ts:153-165).  The engine borrows the parameters of a loaded `WhisperTextDecoder`.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np

from . import core, lib
from .core import Tensor
from .model_utils.whisper import WhisperTextDecoder

KD_ACT_NONE, KD_ACT_GELU = 0, 1


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


def _rows(t: Tensor, a: int, b: int) -> Tensor:
    return t.slice([slice(a, b)] + [slice(None)] * (t.ndim - 1))


class WhisperDecoderEngine:
    def __init__(self, decoder: WhisperTextDecoder, max_batch: int):
        cfg = decoder.config
        if cfg.dtype != "bfloat16":
            raise ValueError("WhisperDecoderEngine needs a bfloat16 decoder")
        self.dec, self.cfg = decoder, cfg
        self.E, self.H, self.T, self.V = cfg.nTextState, cfg.nTextHead, cfg.nTextCtx, cfg.nVocab
        self.D = self.E // self.H
        if self.D not in (64, 128):
            raise ValueError(f"head_dim {self.D} is not handled by the tensor-core attention kernels (64 or 128)")
        self.B = int(max_batch)
        self.scale = 1.0 / math.sqrt(self.D)
        E = self.E
        # self-attention cache [B,H,T,D] per layer, zero-initialised
        self.k_cache = [core.zeros((self.B, self.H, self.T, self.D), "bfloat16") for _ in decoder.layers]
        self.v_cache = [core.zeros((self.B, self.H, self.T, self.D), "bfloat16") for _ in decoder.layers]
        # weight views: query rows / key+value rows of the packed projections
        self.views = []
        for blk in decoder.layers:
            ca = blk.encoder_attn
            self.views.append({
                "cq_w": _rows(ca.in_proj_weight, 0, E), "cq_b": _rows(ca.in_proj_bias, 0, E),
                "ckv_w": _rows(ca.in_proj_weight, E, 3 * E), "ckv_b": _rows(ca.in_proj_bias, E, 3 * E),
            })
        self.cross = None          # per layer (packed K|V buffer, K view, V view) of the current clips
        self.pos = 0
        self.cur_B = 0

    # ------------------------------------------------------------------ encoder side, once per clip
    def set_audio(self, xa: Tensor) -> None:
        """xa [B,S,E] bf16 (the audio encoder's output).  Projects keys and values of every layer's
        cross attention; resets the text position."""
        if xa.dtype != "bfloat16" or xa.ndim != 3 or xa.shape[2] != self.E or xa.shape[0] > self.B:
            raise ValueError(f"xa must be bf16 [B<={self.B}, S, {self.E}]")
        B, S, E = xa.shape
        self._drop_cross()
        self.cross = []
        for vw in self.views:
            kv = core.empty((B, S, 2 * E), "bfloat16")
            lib.call("kd_linear_bf16_bias", _r(xa), _r(vw["ckv_w"]), _r(vw["ckv_b"]), None, KD_ACT_NONE, _r(kv))
            h = kv.view(B, S, 2 * self.H, self.D)
            k = h.slice([slice(None), slice(None), slice(0, self.H), slice(None)]).permute([0, 2, 1, 3])        # [B,H,S,D]
            v = h.slice([slice(None), slice(None), slice(self.H, 2 * self.H), slice(None)]).permute([0, 2, 1, 3])
            h.dispose()
            self.cross.append((kv, k, v))
        self.pos, self.cur_B, self.S_enc = 0, B, S

    def _drop_cross(self) -> None:
        if self.cross:
            for kv, k, v in self.cross:
                for t in (k, v, kv):
                    t.dispose()
        self.cross = None

    # ------------------------------------------------------------------ text side
    def _forward(self, tokens: np.ndarray, all_logits: bool) -> Tensor:
        if self.cross is None:
            raise ValueError("set_audio() first")
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        B, Tn = tokens.shape
        if B != self.cur_B:
            raise ValueError(f"{B} token rows for {self.cur_B} clips")
        off = self.pos
        if off + Tn > self.T:
            raise ValueError(f"positions {off}..{off + Tn} exceed the decoder context of {self.T}")
        if Tn > 1 and off != 0:
            raise ValueError("several positions at once only at the start of the text (the prompt); then one per step")
        E, H, D, dec = self.E, self.H, self.D, self.dec
        e = lambda *shape: core.empty(shape, "bfloat16")  # noqa: E731
        ids = Tensor(tokens)
        emb = dec.embed_tokens(ids)
        pe = dec.embed_positions.weight.slice([slice(off, off + Tn), slice(None)])
        x = core.add(emb, pe)
        for t in (ids, emb, pe):
            t.dispose()
        ctx_self = off + Tn
        for li, blk in enumerate(dec.layers):
            vw = self.views[li]
            sa, ca = blk.self_attn, blk.encoder_attn
            # ---- self attention with the cache
            y = blk.self_attn_layer_norm(x)
            qkv = e(B, Tn, 3 * E)
            lib.call("kd_linear_bf16_bias", _r(y), _r(sa.in_proj_weight), _r(sa.in_proj_bias), None, KD_ACT_NONE, _r(qkv))
            heads = qkv.view(B, Tn, 3 * H, D)
            q, kn, vn = (heads.slice([slice(None), slice(None), slice(j * H, (j + 1) * H), slice(None)]).permute([0, 2, 1, 3])
                         for j in range(3))                                   # [B,H,Tn,D] views
            kc = self.k_cache[li].slice([slice(0, B), slice(None), slice(None), slice(None)])
            vc = self.v_cache[li].slice([slice(0, B), slice(None), slice(None), slice(None)])
            kdst = kc.slice([slice(None), slice(None), slice(off, off + Tn), slice(None)])
            vdst = vc.slice([slice(None), slice(None), slice(off, off + Tn), slice(None)])
            core.copy_(kdst, kn)
            core.copy_(vdst, vn)
            attn = e(B, Tn, E)
            o = attn.view(B, Tn, H, D).permute([0, 2, 1, 3])
            if Tn == 1:
                lib.call("kd_attention_decode", _r(q), _r(kc), _r(vc), None, ctx_self, ctypes.c_float(self.scale), 0, _r(o))
            else:
                kp = kc.slice([slice(None), slice(None), slice(0, ctx_self), slice(None)])
                vp = vc.slice([slice(None), slice(None), slice(0, ctx_self), slice(None)])
                lib.call("kd_flash_attention", _r(q), _r(kp), _r(vp), _r(o), ctypes.c_float(self.scale), 1)
                kp.dispose()
                vp.dispose()
            x1 = e(B, Tn, E)
            lib.call("kd_linear_bf16_bias", _r(attn), _r(sa.out_proj.weight), _r(sa.out_proj.bias), _r(x), KD_ACT_NONE, _r(x1))
            # ---- cross attention on the clip's cached keys / values
            yc = blk.encoder_attn_layer_norm(x1)
            qc = e(B, Tn, E)
            lib.call("kd_linear_bf16_bias", _r(yc), _r(vw["cq_w"]), _r(vw["cq_b"]), None, KD_ACT_NONE, _r(qc))
            qch = qc.view(B, Tn, H, D).permute([0, 2, 1, 3])
            ac = e(B, Tn, E)
            oc = ac.view(B, Tn, H, D).permute([0, 2, 1, 3])
            _, ck, cv = self.cross[li]
            if Tn == 1:
                lib.call("kd_attention_decode", _r(qch), _r(ck), _r(cv), None, self.S_enc, ctypes.c_float(self.scale), 0, _r(oc))
            else:
                lib.call("kd_flash_attention", _r(qch), _r(ck), _r(cv), _r(oc), ctypes.c_float(self.scale), 0)
            x2 = e(B, Tn, E)
            lib.call("kd_linear_bf16_bias", _r(ac), _r(ca.out_proj.weight), _r(ca.out_proj.bias), _r(x1), KD_ACT_NONE, _r(x2))
            # ---- MLP
            y2 = blk.final_layer_norm(x2)
            hmid = e(B, Tn, 4 * E)
            lib.call("kd_linear_bf16_bias", _r(y2), _r(blk.fc1.weight), _r(blk.fc1.bias), None, KD_ACT_GELU, _r(hmid))
            x3 = e(B, Tn, E)
            lib.call("kd_linear_bf16_bias", _r(hmid), _r(blk.fc2.weight), _r(blk.fc2.bias), _r(x2), KD_ACT_NONE, _r(x3))
            for t in (y, qkv, heads, q, kn, vn, kc, vc, kdst, vdst, attn, o, x1, yc, qc, qch, ac, oc, x2, y2, hmid, x):
                t.dispose()
            x = x3
        self.pos = off + Tn
        # logits = layer_norm(x) @ embed_tokens.weight^T (decoder.ts:250-257), fp32; last position unless all are asked for
        xs = x if all_logits else x.slice([slice(None), slice(Tn - 1, Tn), slice(None)])
        y = dec.layer_norm(xs)
        rows = y.shape[0] * y.shape[1]
        y2d = core.contiguous(y).view(rows, E) if not y.isContiguous() else y.view(rows, E)
        logits = core.empty((rows, self.V), "float32")
        # the `matmul` key with transposeB (what `linear` issues): any vocabulary size (51865 is odd),
        # fp32 result from bf16 operands
        cfg = lib.kd_matmul_cfg()
        cfg.M, cfg.N, cfg.K = rows, self.V, E
        cfg.transpose_a, cfg.transpose_b, cfg.alpha, cfg.beta, cfg.has_c = 0, 1, 1.0, 0.0, 0
        lib.call("kd_matmul", ctypes.byref(cfg), _r(y2d), _r(dec.embed_tokens.weight), None, _r(logits))
        out = logits.view(B, y.shape[1], self.V)
        for t in (y2d, y, x) + (() if xs is x else (xs,)):
            t.dispose()
        return out

    def forward(self, tokens: np.ndarray, all_logits: bool = False) -> Tensor:
        """The prompt: tokens [B,T] at positions 0..T-1.  Returns fp32 logits [B,1,V] of the last
        position (or [B,T,V])."""
        return self._forward(tokens, all_logits)

    def step(self, tokens: np.ndarray) -> Tensor:
        """One new token per clip at the next position.  Returns fp32 logits [B,1,V]."""
        tokens = np.asarray(tokens).reshape(self.cur_B, 1)
        return self._forward(tokens, False)

    def generate_greedy(self, prompt: np.ndarray, steps: int) -> np.ndarray:
        """Greedy continuation of `prompt` [B,T]: int64 [B, steps]."""
        logits = self.forward(prompt)
        out = np.empty((prompt.shape[0], steps), np.int64)
        for s in range(steps):
            flat = logits.view(prompt.shape[0], self.V)
            tok = core.argmax(flat, -1).dataAsync().astype(np.int64)
            flat.dispose()
            logits.dispose()
            out[:, s] = tok
            if s + 1 < steps:
                logits = self.step(tok)
        return out

    def dispose(self) -> None:
        self._drop_cross()
