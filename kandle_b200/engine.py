"""Fused bf16 fast path for Qwen3-architecture decoders: tensor-core GEMMs with fused epilogues,
tcgen05 flash attention, split-KV decode attention and a CUDA-graph decode step.

It computes what `Qwen3ForCausalLM.forwardWithKVCache` + greedy argmax compute on the eager path
(packages/model-utils/src/qwen3/for_causal_lm.ts:170-194,475-508), with the ~41 backend calls per
layer collapsed into 7 (prefill) / 3 (decode) kernels and no intermediate copies:

  prefill, per layer     rms_norm -> QKV GEMM (epilogue: q/k-norm+RoPE+cache write) -> flash attention ->
                         o_proj GEMM (+residual) -> rms_norm -> gate/up GEMM (SiLU*up epilogue) ->
                         down GEMM (+residual)
  decode step, per layer norm+RoPE+cache write (sums the QKV split-K partials) -> split-KV attention ->
                         one persistent kernel: o_proj -> residual+rms_norm -> gate/up with SiLU*up
                         -> down -> residual+rms_norm -> the NEXT layer's QKV partials
                         (tensor parallel: the same steps as separate kernels, with all-reduces)
  The decode step reads the write position / context length from device memory, so one captured
  graph is replayed for every step.

Numerics: weights and GEMM / attention operands are bf16, every accumulation is fp32, and the
residual stream and the logits are kept in fp32 (bf16 rounding of the residual at every layer is
the largest avoidable error source; it costs 2 extra bytes per hidden element per layer).

All activations live in buffers allocated once per (batch, sequence) shape; 180 GB of HBM makes a
static workspace the simple choice.
"""
from __future__ import annotations

import ctypes
import os
import math

import numpy as np

from . import core, lib, parallel
from .core import Tensor
from .model_utils.qwen3 import Qwen3Config


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


def interleave_gate_up(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """[I,K] gate and up weights -> [2I,K] with 16 gate rows followed by the 16 matching up rows,
    the row order the SiLU*up GEMM epilogue and kd_swiglu expect."""
    I, K = gate.shape
    assert I % 16 == 0 and up.shape == gate.shape
    return np.stack([gate.reshape(I // 16, 16, K), up.reshape(I // 16, 16, K)], axis=1).reshape(2 * I, K)


class RandomInit:
    """Stands in for a weight dictionary: every linear / embedding weight is drawn N(0, std) on the
    device by the `randn` kernel (Philox4x32-10 keyed by `seed`), RMSNorm weights are ones as the
    modules construct them (packages/core/src/nn/modules/normalization/RMSNorm.ts:85).  Each tensor
    of the FULL model owns a fixed range of the generator's counter space, and a tensor-parallel
    rank draws exactly the rows / columns it owns, so every rank count sees the same model and no
    weight ever exists on the host."""

    def __init__(self, seed: int = 1234, std: float = 0.02):
        self.seed, self.std = int(seed), float(std)


class Qwen3Engine:
    def __init__(self, cfg: Qwen3Config, weights, max_batch: int, max_seq_len: int, tp_size: int = 1, tp_rank: int = 0,
                 paged: bool = False, page_table: np.ndarray | None = None):
        """weights: HuggingFace-style names -> float32 arrays (rounded to bf16 on upload), or a
        RandomInit.  With tp_size > 1 a weight dictionary is this rank's tensor-parallel slice
        (parallel.shard_qwen3_weights; a RandomInit draws rank `tp_rank`'s slice itself), cfg
        describes the FULL model, and the library's communicator must have been initialised: the
        partial outputs of o_proj and down_proj are all-reduced before the residual add.
        paged=True keeps the KV cache in pools of 128-position pages [pages,Hkv,128,D] per layer,
        addressed through a block table int32 [max_batch, ceil(max_seq_len / 128)] (`page_table`, by
        default a fixed shuffle of all pages): same cache semantics as the contiguous StaticKVCache
        (packages/model-utils/src/kv-cache.ts:164-212), same tokens."""
        self.cfg = cfg
        self.tp = int(tp_size)
        self.B, self.max_seq_len = max_batch, max_seq_len
        c = cfg
        if c.numAttentionHeads % self.tp or c.numKeyValueHeads % self.tp or c.intermediateSize % self.tp:
            raise ValueError(f"heads / intermediate size do not divide over {self.tp} ranks")
        self.H, self.D, self.Hq, self.Hkv, self.I, self.V, self.L = (c.hiddenSize, c.headDim, c.numAttentionHeads // self.tp,
                                                                     c.numKeyValueHeads // self.tp,
                                                                     c.intermediateSize // self.tp, c.vocabSize,
                                                                     c.numHiddenLayers)
        if self.D not in (64, 128):
            raise ValueError("the fused engine supports head_dim 64 or 128")
        self.nqkv = (self.Hq + 2 * self.Hkv) * self.D
        bf = lambda a: Tensor(np.ascontiguousarray(a, dtype=np.float32), dtype="bfloat16")  # noqa: E731
        self.layers = []
        if isinstance(weights, RandomInit):
            self._random_weights(weights, int(tp_rank))
        else:
            self.embed = bf(weights["model.embed_tokens.weight"])
            self.final_norm = bf(weights["model.norm.weight"])
        for i in range(self.L if not isinstance(weights, RandomInit) else 0):
            p = f"model.layers.{i}."
            self.layers.append({
                "in_norm": bf(weights[p + "input_layernorm.weight"]),
                "post_norm": bf(weights[p + "post_attention_layernorm.weight"]),
                "wqkv": bf(np.concatenate([weights[p + "self_attn.q_proj.weight"], weights[p + "self_attn.k_proj.weight"],
                                           weights[p + "self_attn.v_proj.weight"]], axis=0)),
                "q_norm": bf(weights[p + "self_attn.q_norm.weight"]),
                "k_norm": bf(weights[p + "self_attn.k_norm.weight"]),
                "wo": bf(weights[p + "self_attn.o_proj.weight"]),
                "wgu": bf(interleave_gate_up(weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"])),
                "wdown": bf(weights[p + "mlp.down_proj.weight"]),
            })
        half = self.D // 2
        inv = np.array([1.0 / math.pow(c.ropeTheta, i / half) for i in range(half)], dtype=np.float32)  # rope.ts:159-171
        self.inv_freq = Tensor(inv, dtype="float32")
        self.paged = bool(paged)
        if self.paged:
            per_seq = (max_seq_len + 127) // 128
            n_pages = self.B * per_seq
            if page_table is None:
                page_table = np.random.Generator(np.random.PCG64(7)).permutation(n_pages).reshape(self.B, per_seq)
            page_table = np.ascontiguousarray(page_table, dtype=np.int32)
            if page_table.shape != (self.B, per_seq) or page_table.min() < 0 or len(np.unique(page_table)) != n_pages:
                raise ValueError(f"page_table must hold {n_pages} distinct page indices in a [{self.B},{per_seq}] array")
            n_pool = int(page_table.max()) + 1
            self.block_table = Tensor(page_table)
            # pools [pages,Hkv,128,D] per layer, zero-initialised like the contiguous cache
            self.k_cache = [core.zeros((n_pool, self.Hkv, 128, self.D), "bfloat16") for _ in range(self.L)]
            self.v_cache = [core.zeros((n_pool, self.Hkv, 128, self.D), "bfloat16") for _ in range(self.L)]
        else:
            self.block_table = None
            # KV cache [B,Hkv,maxS,D] per layer, zero-initialised (kv-cache.ts:123-130)
            self.k_cache = [core.zeros((self.B, self.Hkv, max_seq_len, self.D), "bfloat16") for _ in range(self.L)]
            self.v_cache = [core.zeros((self.B, self.Hkv, max_seq_len, self.D), "bfloat16") for _ in range(self.L)]
        self.scale = 1.0 / math.sqrt(self.D)
        self._prefill_bufs = {}
        self._decode = None
        self.pos = 0
        self.use_pdl = True
        self.use_early_kv = os.environ.get("KD_EARLY_KV", "1") != "0"
        # decode: run o_proj .. next layer's QKV as one persistent kernel per layer (kd_decode_layer_chain);
        # tensor parallelism needs an all-reduce after o_proj and down_proj, so it keeps separate kernels
        self.use_chain = self.tp == 1 and self.H <= 4096
        # ... and further, through the next layer's q/k-norm + RoPE + cache write, in four phases
        # (kd_decode_layer_fused): two launches per layer and decode step
        # (tensor parallel: the form of that kernel that exchanges the partial sums of o_proj and down_proj
        # with its peers inside the kernel, when the peer buffers are connected)
        self.use_fused_layer = self.D == 128 and self.H <= 8192
        # tensor parallel decode: sum the partial outputs over ranks through mapped peer memory when
        # the host program has connected the peer buffers (parallel.init_peer_buffers), else NCCL
        self.use_p2p = True
        self.sampler = None   # None: greedy argmax; else dict(temperature, top_k, top_p, rng), see set_sampler

    def _random_weights(self, init: RandomInit, rank: int) -> None:
        c, tp, D = self.cfg, self.tp, self.D
        Hq_full, Hkv_full, I_full, H = c.numAttentionHeads, c.numKeyValueHeads, c.intermediateSize, self.H
        state = {"offset": 0}

        def draw(out: Tensor, full_rows: int, full_cols: int, row0: int = 0, col0: int = 0, reserve: bool = True) -> None:
            """`out` = the [rows, cols] block at (row0, col0) of a full_rows x full_cols weight whose
            numbers start at the current generator offset."""
            lib.call("kd_randn", _r(out), ctypes.c_uint64(init.seed), ctypes.c_uint32(state["offset"] & 0xFFFFFFFF),
                     ctypes.c_float(0.0), ctypes.c_float(init.std), row0, col0, full_cols)
            if reserve:
                state["offset"] += (full_rows * full_cols + 1) // 2

        e = lambda *shape: core.empty(shape, "bfloat16")  # noqa: E731
        self.embed = e(self.V, H)
        draw(self.embed, self.V, H)
        self.final_norm = core.ones((H,), "bfloat16")
        for _ in range(self.L):
            wqkv = e(self.nqkv, H)
            r0 = 0
            for heads_full, heads_local in ((Hq_full, self.Hq), (Hkv_full, self.Hkv), (Hkv_full, self.Hkv)):   # q, k, v
                part = wqkv.slice([slice(r0, r0 + heads_local * D), slice(None)])
                draw(part, heads_full * D, H, row0=rank * heads_local * D)
                part.dispose()
                r0 += heads_local * D
            wo = e(H, self.Hq * D)
            draw(wo, H, Hq_full * D, col0=rank * self.Hq * D)
            wgu = e(2 * self.I, H)            # drawn directly in the interleaved row order (16 gate rows, 16 up rows)
            draw(wgu, 2 * I_full, H, row0=rank * 2 * self.I)
            wdown = e(H, self.I)
            draw(wdown, H, I_full, col0=rank * self.I)
            self.layers.append({
                "in_norm": core.ones((H,), "bfloat16"), "post_norm": core.ones((H,), "bfloat16"), "wqkv": wqkv,
                "q_norm": core.ones((D,), "bfloat16"), "k_norm": core.ones((D,), "bfloat16"), "wo": wo, "wgu": wgu, "wdown": wdown,
            })

    # ------------------------------------------------------------------ helpers
    def _linear(self, x, w, out, resid=None, epi=0):
        lib.call("kd_linear_bf16", _r(x), _r(w), _r(resid), epi, _r(out))

    def _norm(self, x, w, out, resid=None, sum_out=None):
        lib.call("kd_add_rmsnorm", _r(x), _r(resid), _r(w), ctypes.c_float(self.cfg.rmsNormEps), _r(sum_out), _r(out))

    def set_sampler(self, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0) -> None:
        """Next tokens are drawn on the device (kd_sample: temperature, top-k, top-p, multinomial, the
        reference's `sample` of packages/model-utils/src/sampling/index.ts:103-238) instead of the
        greedy argmax.  The uniform numbers come from a seeded host generator, one per sequence and
        step (128 bytes uploaded per step).  set_sampler(None) restores greedy decoding."""
        self.dispose()       # a captured decode graph holds the old choice
        if temperature is None:
            self.sampler = None
            return
        self.sampler = {"temperature": float(temperature), "top_k": int(top_k), "top_p": float(top_p),
                        "rng": np.random.Generator(np.random.PCG64(seed))}

    def _next_tokens(self, logits2d: Tensor, uniforms, out_ids: Tensor) -> None:
        if self.sampler is None:
            lib.call("kd_argmax", _r(logits2d), _r(out_ids))
        else:
            sp = self.sampler
            lib.call("kd_sample", _r(logits2d), ctypes.c_double(sp["temperature"]), sp["top_k"], ctypes.c_double(sp["top_p"]), 1,
                     _r(uniforms), _r(out_ids), None)

    def _fresh_uniforms(self, t: Tensor) -> None:
        u = self.sampler["rng"].random(t.shape[0], dtype=np.float32)
        core._backend().upload(t._handle, u)

    def _allreduce(self, t) -> None:
        lib.call("kd_allreduce_sum", _r(t))

    def _reduce_add_norm(self, d: dict, partials, norm_w, resid, sum_out) -> None:
        """sum_out = resid + (sum over ranks and splits of `partials`); d["x"] = RMSNorm(sum_out).
        Tensor parallel with mapped peer buffers: one kernel does the sum over ranks through peer
        memory (kd_allreduce_add_rmsnorm); otherwise the library all-reduce followed by the fused
        add + norm kernel."""
        if self.tp > 1 and d["p2p"]:
            lib.call("kd_allreduce_add_rmsnorm", _r(partials), _r(resid), _r(norm_w), ctypes.c_float(self.cfg.rmsNormEps),
                     _r(sum_out), _r(d["x"]))
            return
        if self.tp > 1:
            self._allreduce(partials)
        self._norm(partials, norm_w, d["x"], resid=resid, sum_out=sum_out)

    def kv_bytes_per_token(self) -> int:
        return 2 * self.L * self.Hkv * self.D * 2

    # ------------------------------------------------------------------ prefill
    def _bufs(self, B: int, S: int) -> dict:
        key = (B, S)
        if key not in self._prefill_bufs:
            T = B * S
            e = lambda *shape: core.empty(shape, "bfloat16")  # noqa: E731
            self._prefill_bufs = {key: {
                "ids": core.empty((T,), "int32"), "emb": e(T, self.H), "h": core.empty((T, self.H), "float32"),
                "h1": core.empty((T, self.H), "float32"), "x": e(T, self.H),
                "part": e(T, self.H) if self.tp > 1 else None,
                "qkv": e(T, self.nqkv), "q": e(B, S, self.Hq, self.D), "attn": e(B, S, self.Hq, self.D),
                "act": e(T, self.I), "cos": core.empty((S, self.D // 2), "float32"),
                "sin": core.empty((S, self.D // 2), "float32"), "last": core.empty((B, self.H), "float32"), "xl": e(B, self.H),
                "logits": core.empty((1, B, self.V), "float32"), "tok": core.empty((B,), "int64"),
                "uniforms": core.zeros((B,), "float32"),
                # paged cache: the prompt's K/V of one layer, contiguous, before they are scattered into pages
                "kt": e(B, self.Hkv, S, self.D) if self.paged else None, "vt": e(B, self.Hkv, S, self.D) if self.paged else None,
            }}
        return self._prefill_bufs[key]

    def prefill(self, ids, all_logits: bool = False):
        """ids: host int32 array [B,S] (uploaded here) or an int32 device Tensor [B,S].  Fills the KV
        cache for positions [0,S) and returns the greedy next token per sequence as a device int64
        Tensor [B] (plus fp32 logits for every position when all_logits is set, which is what the
        unmodified model code computes)."""
        if isinstance(ids, Tensor):
            B, S = ids.shape
            ids_t = ids.view(B * S)
        else:
            ids = np.ascontiguousarray(ids, dtype=np.int32)
            B, S = ids.shape
            ids_t = None
        if B > self.B or S > self.max_seq_len:
            raise ValueError(f"prefill of {B}x{S} exceeds the engine's {self.B}x{self.max_seq_len}")
        w = self._bufs(B, S)
        if ids_t is None:
            core._backend().upload(w["ids"]._handle, ids.reshape(-1))
            ids_t = w["ids"]
        c = self.cfg
        T = B * S
        core._kernel("index_select")(self.embed._handle, ids_t._handle, {"dim": 0}, w["emb"]._handle)
        core.copy_(w["h"], w["emb"])                       # bf16 embedding rows -> fp32 residual stream
        lib.call("kd_rope_table", _r(self.inv_freq), None, 0, S, _r(w["cos"]), _r(w["sin"]))
        q_bhsd = w["q"].permute([0, 2, 1, 3])
        o_bhsd = w["attn"].permute([0, 2, 1, 3])
        attn2d = w["attn"].view(T, self.Hq * self.D)
        h, h1 = w["h"], w["h1"]
        table = self.block_table.slice([slice(0, B), slice(None)]) if self.paged else None
        for li, lw in enumerate(self.layers):
            if self.paged:
                # the prompt's K/V go to a contiguous buffer that the attention reads, then into the pages
                kc, vc = w["kt"].slice(":, :, :, :"), w["vt"].slice(":, :, :, :")
            else:
                kc = self.k_cache[li].slice([slice(0, B), slice(None), slice(None), slice(None)])
                vc = self.v_cache[li].slice([slice(0, B), slice(None), slice(None), slice(None)])
            if self.tp == 1 or li == 0:
                self._norm(h, lw["in_norm"], w["x"])     # (tensor parallel: later layers get x from the fused add+norm)
            if self.D == 128:
                # QKV GEMM whose epilogue does q/k-norm + RoPE + the KV-cache write
                lib.call("kd_qkv_linear_norm_rope_cachewrite", _r(w["x"]), _r(lw["wqkv"]), _r(lw["q_norm"]), _r(lw["k_norm"]),
                         ctypes.c_float(c.rmsNormEps), _r(w["cos"]), _r(w["sin"]), _r(kc), _r(vc), 0, _r(w["q"]))
            else:
                self._linear(w["x"], lw["wqkv"], w["qkv"])
                lib.call("kd_qkv_norm_rope_cachewrite", _r(w["qkv"]), _r(lw["q_norm"]), _r(lw["k_norm"]),
                         ctypes.c_float(c.rmsNormEps), _r(w["cos"]), _r(w["sin"]), _r(kc), _r(vc), None, 0, _r(w["q"]))
            kp, vp = kc.slice(f":, :, :{S}, :"), vc.slice(f":, :, :{S}, :")
            lib.call("kd_flash_attention", _r(q_bhsd), _r(kp), _r(vp), _r(o_bhsd), ctypes.c_float(self.scale), 1)
            if self.paged:
                lib.call("kd_kv_pages_write", _r(kp), _r(vp), _r(self.k_cache[li]), _r(self.v_cache[li]), _r(table), 0)
            if self.tp == 1:
                self._linear(attn2d, lw["wo"], h1, resid=h, epi=1)
                self._norm(h1, lw["post_norm"], w["x"])
                self._linear(w["x"], lw["wgu"], w["act"], epi=2)
                self._linear(w["act"], lw["wdown"], h, resid=h1, epi=1)
            else:
                # tensor parallel: each rank holds a partial sum of o_proj / down_proj (bf16), summed
                # over ranks before the residual add (fused with the following RMSNorm)
                self._linear(attn2d, lw["wo"], w["part"])
                self._allreduce(w["part"])
                self._norm(w["part"], lw["post_norm"], w["x"], resid=h, sum_out=h1)
                self._linear(w["x"], lw["wgu"], w["act"], epi=2)
                self._linear(w["act"], lw["wdown"], w["part"])
                self._allreduce(w["part"])
                nxt = self.layers[li + 1]["in_norm"] if li + 1 < self.L else self.final_norm
                self._norm(w["part"], nxt, w["x"], resid=h1, sum_out=h)
            for t in (kc, vc, kp, vp):
                t.dispose()
        # tied lm_head on the last position of every sequence (select commutes with the row-wise matmul)
        h3 = h.view(B, S, self.H)
        last = h3.select(1, S - 1)
        core.copy_(w["last"], last)
        self._norm(w["last"], self.final_norm, w["xl"])
        lib.call("kd_linear_bf16_skinny", _r(w["xl"]), _r(self.embed), 0, _r(w["logits"]))
        lg = w["logits"].view(B, self.V)
        if self.sampler is not None:
            self._fresh_uniforms(w["uniforms"])
        self._next_tokens(lg, w["uniforms"], w["tok"])
        lg.dispose()
        full = None
        if all_logits:
            xa = core.empty((T, self.H), "bfloat16")
            self._norm(h, self.final_norm, xa)
            full = core.empty((B, S, self.V), "float32")
            self._linear(xa, self.embed, full)
            xa.dispose()
        for t in (q_bhsd, o_bhsd, attn2d, h3, last):
            t.dispose()
        if table is not None:
            table.dispose()
        self.pos = S
        self.cur_B = B
        return (w["tok"], full) if all_logits else w["tok"]

    # ------------------------------------------------------------------ decode
    def _decode_state(self, B: int) -> dict:
        if self._decode is not None and self._decode["B"] == B:
            return self._decode
        self.dispose()        # another batch size: the captured graph of the old state goes with it
        def splits(n, k):
            s = ctypes.c_int(0)
            lib.call("kd_linear_bf16_skinny_splits", ctypes.c_int64(n), ctypes.c_int64(k), ctypes.byref(s))
            return s.value
        e = lambda *shape: core.empty(shape, "bfloat16")  # noqa: E731
        f = lambda *shape: core.empty(shape, "float32")  # noqa: E731
        def chain_splits(n, k):
            s = ctypes.c_int(0)
            lib.call("kd_decode_layer_chain_splits", ctypes.c_int64(n), ctypes.c_int64(k), ctypes.byref(s))
            return s.value
        p2p = self.tp > 1 and self.use_p2p and parallel.peer_buffers_ready()
        d = {
            "B": B, "graph": None, "chain": self.use_chain,
            # (tensor parallel: fp32 partial sums of all sequences must fit one 2 MiB exchange slot)
            "fused": self.use_fused_layer and (self.tp == 1 or (p2p and B * self.H * 4 <= (2 << 20))),
            "p2p": p2p,
            "scalars": core.zeros((2,), "int32"),           # [write position, context length]
            "ids": core.zeros((B,), "int64"), "emb": e(B, self.H), "h": f(B, self.H), "h1": f(B, self.H), "x": e(B, self.H),
            # a projection whose suggested split factor is 1 writes bf16 directly, otherwise fp32 partials
            "qkv_p": (e(B, self.nqkv) if splits(self.nqkv, self.H) == 1 else f(splits(self.nqkv, self.H), B, self.nqkv)),
            "q": e(B, 1, self.Hq, self.D),
            "attn": e(B, 1, self.Hq, self.D), "o_p": f(splits(self.H, self.Hq * self.D), B, self.H),
            "act": e(B, self.I),
            "down_p": f(splits(self.H, self.I), B, self.H), "logits": f(1, B, self.V),
            "cos": f(1, self.D // 2), "sin": f(1, self.D // 2), "uniforms": core.zeros((B,), "float32"),
        }
        if self.use_chain and not self.use_fused_layer:
            d["qkv_p"].dispose()
            d["qkv_p"] = f(chain_splits(self.nqkv, self.H), B, self.nqkv)
        d["pos"] = d["scalars"].slice([slice(0, 1)])
        d["ctx"] = d["scalars"].slice([slice(1, 2)])
        self._decode = d
        return d

    def _enqueue_decode_step(self, d: dict) -> None:
        """One decode step for d['ids'] at device position d['pos']; leaves the next ids in d['ids']."""
        # every kernel below starts with a grid-dependency wait; 2: the decode attention may fetch the K/V
        # tiles of earlier positions before its wait (this step writes one new cache row per layer, and
        # the context length dates from the previous step)
        lib.call("kd_set_pdl", (2 if self.use_early_kv else 1) if self.use_pdl else 0)
        try:
            self._decode_step_kernels(d)
        finally:
            lib.call("kd_set_pdl", 0)

    def _decode_step_kernels(self, d: dict) -> None:
        c, B = self.cfg, d["B"]
        eps = ctypes.c_float(c.rmsNormEps)
        core._kernel("index_select")(self.embed._handle, d["ids"]._handle, {"dim": 0}, d["emb"]._handle)
        core.copy_(d["h"], d["emb"])
        lib.call("kd_rope_table", _r(self.inv_freq), _r(d["pos"]), 0, 1, _r(d["cos"]), _r(d["sin"]))
        q_bh1d = d["q"].permute([0, 2, 1, 3])
        o_bh1d = d["attn"].permute([0, 2, 1, 3])
        attn2d = d["attn"].view(B, self.Hq * self.D)
        h, h1 = d["h"], d["h1"]
        self._norm(h, self.layers[0]["in_norm"], d["x"])
        table = self.block_table.slice([slice(0, B), slice(None)]) if self.paged else None

        def cache_of(layer):
            if self.paged:      # whole pools; the block table selects the pages of the B sequences
                return self.k_cache[layer].slice(":, :, :, :"), self.v_cache[layer].slice(":, :, :, :")
            return (self.k_cache[layer].slice([slice(0, B), slice(None), slice(None), slice(None)]),
                    self.v_cache[layer].slice([slice(0, B), slice(None), slice(None), slice(None)]))

        for li, lw in enumerate(self.layers):
            kc, vc = cache_of(li)
            if li == 0 or not (d["chain"] or d["fused"]):
                lib.call("kd_linear_bf16_skinny", _r(d["x"]), _r(lw["wqkv"]), 0, _r(d["qkv_p"]))
            if li == 0 or not d["fused"]:
                if self.paged:
                    lib.call("kd_qkv_norm_rope_cachewrite_paged", _r(d["qkv_p"]), _r(lw["q_norm"]), _r(lw["k_norm"]), eps, _r(d["cos"]),
                             _r(d["sin"]), _r(kc), _r(vc), _r(table), _r(d["pos"]), 0, _r(d["q"]))
                else:
                    lib.call("kd_qkv_norm_rope_cachewrite", _r(d["qkv_p"]), _r(lw["q_norm"]), _r(lw["k_norm"]), eps, _r(d["cos"]),
                             _r(d["sin"]), _r(kc), _r(vc), _r(d["pos"]), 0, _r(d["q"]))
            if self.paged:
                lib.call("kd_attention_decode_paged", _r(q_bh1d), _r(kc), _r(vc), _r(table), _r(d["ctx"]), 0, ctypes.c_float(self.scale), 0,
                         _r(o_bh1d))
            else:
                lib.call("kd_attention_decode", _r(q_bh1d), _r(kc), _r(vc), _r(d["ctx"]), 0, ctypes.c_float(self.scale), 0, _r(o_bh1d))
            nxt = self.layers[li + 1]["in_norm"] if li + 1 < self.L else self.final_norm
            if d["fused"]:
                layer_fn = "kd_decode_layer_fused_tp" if self.tp > 1 else "kd_decode_layer_fused"
                if li + 1 < self.L:
                    nl = self.layers[li + 1]
                    kn, vn = cache_of(li + 1)
                    lib.call(layer_fn, _r(attn2d), _r(lw["wo"]), _r(h), _r(lw["post_norm"]), _r(lw["wgu"]),
                             _r(lw["wdown"]), _r(nxt), eps, _r(nl["wqkv"]), _r(nl["q_norm"]), _r(nl["k_norm"]), _r(d["cos"]),
                             _r(d["sin"]), _r(d["pos"]), _r(kn), _r(vn), _r(table), _r(d["q"]), _r(h), None)
                    kn.dispose()
                    vn.dispose()
                else:
                    lib.call(layer_fn, _r(attn2d), _r(lw["wo"]), _r(h), _r(lw["post_norm"]), _r(lw["wgu"]),
                             _r(lw["wdown"]), _r(nxt), eps, None, None, None, None, None, None, None, None, None, None, _r(h), _r(d["x"]))
                kc.dispose()
                vc.dispose()
                continue
            if d["chain"]:
                last = li + 1 == self.L
                lib.call("kd_decode_layer_chain", _r(attn2d), _r(lw["wo"]), _r(h), _r(lw["post_norm"]), _r(lw["wgu"]),
                         _r(lw["wdown"]), _r(nxt), eps, None if last else _r(self.layers[li + 1]["wqkv"]), _r(h1), _r(h),
                         _r(d["x"]), _r(d["act"]), None if last else _r(d["qkv_p"]))
                kc.dispose()
                vc.dispose()
                continue
            lib.call("kd_linear_bf16_skinny", _r(attn2d), _r(lw["wo"]), 0, _r(d["o_p"]))
            self._reduce_add_norm(d, d["o_p"], lw["post_norm"], h, h1)
            lib.call("kd_linear_bf16_skinny", _r(d["x"]), _r(lw["wgu"]), 2, _r(d["act"]))   # SiLU*up in the epilogue
            lib.call("kd_linear_bf16_skinny", _r(d["act"]), _r(lw["wdown"]), 0, _r(d["down_p"]))
            self._reduce_add_norm(d, d["down_p"], nxt, h1, h)
            kc.dispose()
            vc.dispose()
        lib.call("kd_linear_bf16_skinny", _r(d["x"]), _r(self.embed), 0, _r(d["logits"]))
        lg = d["logits"].view(B, self.V)
        self._next_tokens(lg, d["uniforms"], d["ids"])
        lg.dispose()
        lib.call("kd_increment_i32", _r(d["pos"]), 1)
        lib.call("kd_increment_i32", _r(d["ctx"]), 1)
        for t in (q_bh1d, o_bh1d, attn2d):
            t.dispose()
        if table is not None:
            table.dispose()

    def start_decode(self, first_tokens: Tensor, use_graph: bool = True) -> dict:
        """Prepares the decode state after a prefill: next input ids = first_tokens (device int64 [B]),
        write position = prompt length.  With use_graph the step is captured once (after one eager
        warm-up step on a scratch position) and replayed by decode_step()."""
        B = first_tokens.shape[0]
        d = self._decode_state(B)
        if self.pos + 1 > self.max_seq_len:
            raise ValueError("Cache overflow: no room left for decode steps")
        be = core._backend()
        if use_graph and d["graph"] is None:
            # warm-up at the current position: sizes the library's scratch and the allocator's caches
            # (nothing may allocate while capturing); the cache row it writes is overwritten by the
            # first real step, which runs at the same position.
            core.copy_(d["ids"], first_tokens)
            be.upload(d["scalars"]._handle, np.array([self.pos, self.pos + 1], np.int32))
            self._enqueue_decode_step(d)
            lib.call("kd_graph_begin")
            try:
                self._enqueue_decode_step(d)
            finally:
                g = ctypes.c_uint64(0)
                lib.call("kd_graph_end", ctypes.byref(g))
            d["graph"] = g.value
        core.copy_(d["ids"], first_tokens)
        be.upload(d["scalars"]._handle, np.array([self.pos, self.pos + 1], np.int32))
        d["use_graph"] = use_graph
        return d

    def decode_step(self) -> Tensor:
        """Runs one step; returns the device int64 [B] tensor holding the tokens just produced."""
        d = self._decode
        if self.pos + 1 > self.max_seq_len:
            raise ValueError(f"Cache overflow: position {self.pos} but maxSeqLen is {self.max_seq_len}")
        if self.sampler is not None:
            self._fresh_uniforms(d["uniforms"])     # read by the (replayed) sampling kernel of this step
        if d["use_graph"]:
            lib.call("kd_graph_launch", ctypes.c_uint64(d["graph"]))
        else:
            self._enqueue_decode_step(d)
        self.pos += 1
        return d["ids"]

    def generate(self, ids, steps: int, use_graph: bool = True) -> np.ndarray:
        """Generation (greedy, or sampled after set_sampler): prefill + `steps` tokens (the first comes from the prefill).  Returns
        int64 [B, steps] on the host; every step's ids are read back, as the reference does."""
        tok = self.prefill(ids)
        B = tok.shape[0]
        out = np.empty((B, steps), dtype=np.int64)
        out[:, 0] = tok.dataAsync()
        if steps > 1:
            self.start_decode(tok, use_graph)
            for t in range(1, steps):
                out[:, t] = self.decode_step().dataAsync()
        return out

    def dispose(self) -> None:
        if self._decode is not None and self._decode.get("graph"):
            lib.call("kd_graph_destroy", ctypes.c_uint64(self._decode["graph"]))
        self._decode = None
