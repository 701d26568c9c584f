"""CPU oracle (numpy front end) for the transformer-forward hot path of final-kk/kandle.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the
cpu_baseline / reference legs of bench.py.  The shipped package never imports it.

PARITY UNPINNED: the reference ships no golden vectors or runnable tests for this path
and cannot be executed here; see the header of oracle.cpp.

The arithmetic lives in oracle.cpp (compiled to oracle/_build/liboracle.so by
`python oracle/build.py`); this module adds the operator sequencing that the reference
does in TypeScript (model-utils and the composite dispatch handlers).  Citations are
paths inside the reference project.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
import sys
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

c_f32p = ctypes.POINTER(ctypes.c_float)
c_i32p = ctypes.POINTER(ctypes.c_int32)
c_i64p = ctypes.POINTER(ctypes.c_int64)


def build(force: bool = False) -> str:
    """Compile oracle.cpp with g++ (AVX2+FMA, OpenMP)."""
    src = os.path.join(_HERE, "oracle.cpp")
    if not force and os.path.exists(_LIB_PATH) and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src):
        return _LIB_PATH
    os.makedirs(os.path.dirname(_LIB_PATH), exist_ok=True)
    cmd = ["g++", "-O3", "-mavx2", "-mfma", "-fopenmp", "-fno-fast-math", "-shared", "-fPIC",
           "-std=c++17", "-o", _LIB_PATH, src]
    subprocess.run(cmd, check=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(int(n))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(c_f32p)


# ----------------------------------------------------------------------------- ops
def linear(x: np.ndarray, w: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    """`linear` composite: x @ w.T, then a separate bias add
    (packages/core/src/dispatch/handlers/composite.ts:55-77)."""
    x = _f32(x)
    w = _f32(w)
    K = x.shape[-1]
    N = w.shape[0]
    assert w.shape[1] == K
    x2 = x.reshape(-1, K)
    out = np.empty((x2.shape[0], N), dtype=np.float32)
    lib().orc_gemm_nt(_p(x2), ctypes.c_int64(K), _p(w), ctypes.c_int64(K), _p(out), ctypes.c_int64(N),
                      ctypes.c_int64(x2.shape[0]), ctypes.c_int64(N), ctypes.c_int64(K),
                      ctypes.c_float(1.0), ctypes.c_float(0.0), None, ctypes.c_int64(0))
    out = out.reshape(*x.shape[:-1], N)
    if bias is not None:
        out = add(out, np.broadcast_to(_f32(bias), out.shape))
    return out


def matmul4d(a: np.ndarray, b: np.ndarray, *, trans_a=False, trans_b=False, alpha=1.0, beta=0.0,
             c: np.ndarray | None = None) -> np.ndarray:
    """General strided batched matmul (MatmulDispatchResult semantics,
    packages/core/src/dispatch/matmulOps.ts:32-125).  `a`/`b` may be arbitrary numpy views with
    up to 4 dims; leading dims broadcast.  The stored last two dims are swapped logically when the
    matching trans flag is set."""
    assert a.dtype == np.float32 and b.dtype == np.float32
    a4 = a.reshape((1,) * (4 - a.ndim) + a.shape) if a.ndim < 4 else a
    b4 = b.reshape((1,) * (4 - b.ndim) + b.shape) if b.ndim < 4 else b
    # reshape of a non-contiguous view may copy; rebuild strides explicitly instead
    def strides4(t):
        st = [s // 4 for s in t.strides]
        return [0] * (4 - t.ndim) + st, (1,) * (4 - t.ndim) + t.shape
    sa, sha = strides4(a)
    sb, shb = strides4(b)
    M, K = (sha[3], sha[2]) if trans_a else (sha[2], sha[3])
    K2, N = (shb[3], shb[2]) if trans_b else (shb[2], shb[3])
    assert K == K2, (sha, shb)
    b0 = max(sha[0], shb[0])
    b1 = max(sha[1], shb[1])
    for d, bd in ((0, b0), (1, b1)):
        if sha[d] == 1 and bd > 1:
            sa[d] = 0
        if shb[d] == 1 and bd > 1:
            sb[d] = 0
    out = np.empty((b0, b1, M, N), dtype=np.float32)
    sa_c = (ctypes.c_int64 * 4)(*sa)
    sb_c = (ctypes.c_int64 * 4)(*sb)
    cp, sc_c = None, (ctypes.c_int64 * 4)(0, 0, 0, 0)
    if c is not None:
        cb = np.ascontiguousarray(np.broadcast_to(c, out.shape), dtype=np.float32)
        cp = _p(cb)
        sc_c = (ctypes.c_int64 * 4)(*[s // 4 for s in cb.strides])
    base_a = ctypes.cast(a.ctypes.data, c_f32p)
    base_b = ctypes.cast(b.ctypes.data, c_f32p)
    lib().orc_matmul4d(base_a, sa_c, int(trans_a), base_b, sb_c, int(trans_b), cp, sc_c, _p(out),
                       ctypes.c_int64(b0), ctypes.c_int64(b1), ctypes.c_int64(M), ctypes.c_int64(N),
                       ctypes.c_int64(K), ctypes.c_float(alpha), ctypes.c_float(beta))
    nd = max(a.ndim, b.ndim)
    return out.reshape(out.shape[4 - nd:])


def sdpa_tile_config(D: int, Sq: int, Skv: int) -> tuple[int, int]:
    bq, bkv = ctypes.c_int(0), ctypes.c_int(0)
    lib().orc_sdpa_tile_config(D, Sq, Skv, ctypes.byref(bq), ctypes.byref(bkv))
    return bq.value, bkv.value


def sdpa(q: np.ndarray, k: np.ndarray, v: np.ndarray, *, scale: float | None = None,
         is_causal: bool = False, block_kv: int = 0) -> np.ndarray:
    """Fused attention kernel reached from `scaled_dot_product_attention` when no mask is given
    (packages/core/src/dispatch/handlers/composite.ts:247-348).  Accepts 2-D, 3-D or 4-D inputs
    like the executor (packages/backend-webgpu/src/kernels/attention/executor.ts:198-220):
    3-D [H,S,D] means batch 1."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    shape = q.shape
    if q.ndim == 2:
        q, k, v = q[None, None], k[None, None], v[None, None]
    elif q.ndim == 3:
        q, k, v = q[None], k[None], v[None]
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)  # composite.ts:272-275
    out = np.empty_like(q)
    lib().orc_sdpa(_p(q), _p(k), _p(v), _p(out), B, Hq, Hkv, Sq, Skv, D, ctypes.c_float(scale),
                   int(bool(is_causal)), int(block_kv))
    return out.reshape(shape)


def rms_norm(x: np.ndarray, w: np.ndarray | None, eps: float = 1e-5) -> np.ndarray:
    x = _f32(x)
    n = x.shape[-1]
    out = np.empty_like(x)
    wp = _p(_f32(w)) if w is not None else None
    lib().orc_rms_norm(_p(x), wp, _p(out), ctypes.c_int64(x.size // n), ctypes.c_int64(n), ctypes.c_float(eps))
    return out


def layer_norm(x: np.ndarray, w: np.ndarray | None, b: np.ndarray | None, eps: float = 1e-5) -> np.ndarray:
    x = _f32(x)
    n = x.shape[-1]
    out = np.empty_like(x)
    wk = _f32(w) if w is not None else None
    bk = _f32(b) if b is not None else None
    lib().orc_layer_norm(_p(x), _p(wk) if wk is not None else None, _p(bk) if bk is not None else None,
                         _p(out), ctypes.c_int64(x.size // n), ctypes.c_int64(n), ctypes.c_float(eps))
    return out


def softmax(x: np.ndarray) -> np.ndarray:
    """softmax over the last dim."""
    x = _f32(x)
    n = x.shape[-1]
    out = np.empty_like(x)
    lib().orc_softmax(_p(x), _p(out), ctypes.c_int64(x.size // n), ctypes.c_int64(n))
    return out


_UNARY = {"neg": 0, "cos": 1, "sin": 2, "silu": 3, "gelu": 4, "abs": 5, "tanh": 6, "sigmoid": 7}


def unary(op: str, x: np.ndarray) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_unary(_UNARY[op], _p(x), _p(out), ctypes.c_int64(x.size))
    return out


def add(a: np.ndarray, b: np.ndarray, alpha: float = 1.0) -> np.ndarray:
    """a + alpha*b in fp32 (packages/backend-webgpu/src/kernels/pointwise/ops.ts:437-444)."""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    if alpha == 1.0:
        return (a + b).astype(np.float32)
    return (a + np.float32(alpha) * b).astype(np.float32)


def mul(a: np.ndarray, b) -> np.ndarray:
    return (np.asarray(a, dtype=np.float32) * np.asarray(b, dtype=np.float32)).astype(np.float32)


def embedding(w: np.ndarray, ids: np.ndarray) -> np.ndarray:
    w = _f32(w)
    flat = np.ascontiguousarray(ids.reshape(-1), dtype=np.int32)
    if flat.size and (flat.min() < 0 or flat.max() >= w.shape[0]):
        raise IndexError("embedding index out of range")
    out = np.empty((flat.size, w.shape[1]), dtype=np.float32)
    lib().orc_index_select_rows(_p(w), flat.ctypes.data_as(c_i32p), _p(out), ctypes.c_int64(flat.size),
                                ctypes.c_int64(w.shape[1]))
    return out.reshape(*ids.shape, w.shape[1])


_PHILOX_M0, _PHILOX_M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32_10(counter: np.ndarray, key0: int, key1: int) -> np.ndarray:
    """Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3",
    SC'11) as the reference states it in WGSL
    (packages/backend-webgpu/src/kernels/random/philox.wgsl.ts:33-113): counter [n,4] uint32 ->
    [n,4] uint32.  Round: (hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0) with (hi0,lo0) = M0*c0,
    (hi1,lo1) = M1*c2; the key grows by (W0, W1) between rounds, not after the last."""
    c = np.array(counter, dtype=np.uint32).reshape(-1, 4).copy()
    k0, k1 = int(key0) & 0xFFFFFFFF, int(key1) & 0xFFFFFFFF
    for _ in range(10):
        p0 = _PHILOX_M0 * c[:, 0].astype(np.uint64)
        p1 = _PHILOX_M1 * c[:, 2].astype(np.uint64)
        n0 = (p1 >> np.uint64(32)).astype(np.uint32) ^ c[:, 1] ^ np.uint32(k0)
        n2 = (p0 >> np.uint64(32)).astype(np.uint32) ^ c[:, 3] ^ np.uint32(k1)
        c = np.stack([n0, p1.astype(np.uint32), n2, p0.astype(np.uint32)], axis=1)
        k0, k1 = (k0 + _PHILOX_W0) & 0xFFFFFFFF, (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return c


def randn(numel: int, seed: int, base_offset: int = 0, first: int = 0) -> np.ndarray:
    """Elements [first, first + numel) of the reference's `randn` stream
    (packages/backend-webgpu/src/kernels/random/shaderBuilder.ts:140-185): element i is member i % 2
    of pair i // 2, counter [pair + base_offset mod 2^32, 0, 0, 0], key = (seed low word, seed high
    word) (random/executor.ts:31-49, packages/types/src/random.ts:77-81); member 0 uses output words
    (x, y), member 1 (z, w); uniform = (w >> 8) * 2^-24 (philox.wgsl.ts:126-129); z = sqrt(-2 ln
    max(u1, 1e-10)) * cos(2 pi u2) in float32 (philox.wgsl.ts:146-154)."""
    i = np.arange(first, first + numel, dtype=np.uint64)
    ctr = np.zeros((numel, 4), np.uint32)
    ctr[:, 0] = ((i >> np.uint64(1)) + np.uint64(base_offset & 0xFFFFFFFF)).astype(np.uint32)   # wraps mod 2^32
    r = philox4x32_10(ctr, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    odd = (i & np.uint64(1)).astype(bool)
    w1 = np.where(odd, r[:, 2], r[:, 0])
    w2 = np.where(odd, r[:, 3], r[:, 1])
    u1 = np.maximum((w1 >> np.uint32(8)).astype(np.float32) * np.float32(5.9604644775390625e-8), np.float32(1e-10))
    u2 = (w2 >> np.uint32(8)).astype(np.float32) * np.float32(5.9604644775390625e-8)
    rad = np.sqrt(np.float32(-2.0) * np.log(u1, dtype=np.float32), dtype=np.float32)
    return (rad * np.cos(np.float32(6.283185307179586) * u2, dtype=np.float32)).astype(np.float32)


def argmax_rows(x: np.ndarray) -> np.ndarray:
    x = _f32(x)
    n = x.shape[-1]
    out = np.empty(x.shape[:-1], dtype=np.int32)
    lib().orc_argmax_rows(_p(x), out.ctypes.data_as(c_i32p), ctypes.c_int64(x.size // n), ctypes.c_int64(n))
    return out


def _softmax_cpu(logits: np.ndarray, temperature: float) -> np.ndarray:
    """softmaxCPU of packages/model-utils/src/sampling/index.ts:260-283: Float32Array storage,
    double arithmetic, sequential double sum of the stored floats."""
    x = np.asarray(logits, dtype=np.float32).astype(np.float64)
    mx = x.max()
    e = np.exp((x - mx) * (1.0 / temperature)).astype(np.float32)
    total = np.cumsum(e.astype(np.float64))[-1]          # cumsum adds left to right, as the JS loop does
    return (e.astype(np.float64) / total).astype(np.float32)


def sample(logits: np.ndarray, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, do_sample: bool = True,
           r: float = 0.5) -> dict:
    """`sample` of packages/model-utils/src/sampling/index.ts:103-238 for one row of logits, with the
    uniform number `r` in place of Math.random() (:291).  Returns token id, logProb and the final
    probability vector."""
    lg = np.asarray(logits, dtype=np.float32).reshape(-1)
    V = lg.size
    order = np.argsort(-lg.astype(np.float64), kind="stable")       # :133, a stable sort: ties keep index order
    if not do_sample:                                                # :138-160
        probs = _softmax_cpu(lg, temperature)
        tok = int(order[0])
        return {"token": tok, "logprob": float(np.log(np.float64(probs[tok]) + 1e-10)), "probs": probs}
    scaled = lg
    if temperature != 1.0:                                           # :167-175
        scaled = (lg.astype(np.float64) * (1.0 / temperature)).astype(np.float32)
    probs = _softmax_cpu(scaled, 1.0)                                # :178
    k_eff = V
    if 0 < top_k < V:                                                # :181-193
        k_eff = top_k
        mask = np.zeros(V, dtype=np.float32)
        mask[order[:top_k]] = 1.0
        probs = (probs * mask).astype(np.float32)
    if top_p < 1.0:                                                  # :196-214
        cum = np.cumsum(probs[order[:k_eff]].astype(np.float64))
        hit = np.nonzero(cum >= top_p)[0]
        cutoff = int(hit[0]) + 1 if hit.size else k_eff
        probs[order[cutoff:]] = 0.0
    total = np.cumsum(probs.astype(np.float64))[-1]                  # :217-222
    if total > 0:
        probs = (probs.astype(np.float64) / total).astype(np.float32)
    cum = np.cumsum(probs.astype(np.float64))                        # :291-306
    hit = np.nonzero(r < cum)[0]
    if hit.size:
        tok = int(hit[0])
    else:
        nz = np.nonzero(probs > 0)[0]
        tok = int(nz[-1]) if nz.size else 0
    return {"token": tok, "logprob": float(np.log(np.float64(probs[tok]) + 1e-10)), "probs": probs}


def stft_power(x: np.ndarray, window: np.ndarray, n_fft: int, hop: int, center: bool = True) -> np.ndarray:
    """|STFT|^2 of a [L] signal -> [T, n_fft/2+1], following the reference's `stft` composite
    (packages/core/src/dispatch/handlers/composite.ts:527-681: constant-mode centre padding, framing,
    window multiply in f32, one-sided transform) and `spectrogram` with power 2
    (audio/functional/spectrogram.ts:63-68: abs, then abs*abs).  The transform itself is evaluated in
    float64 and rounded to f32, i.e. an exactly rounded version of the reference's f32 Bluestein."""
    x = np.asarray(x, dtype=np.float32).reshape(-1)
    w = np.asarray(window, dtype=np.float32)
    pad = n_fft // 2 if center else 0
    xp = np.concatenate([np.zeros(pad, np.float32), x, np.zeros(pad, np.float32)])
    T = 1 + (xp.size - n_fft) // hop
    idx = np.arange(T)[:, None] * hop + np.arange(n_fft)[None, :]
    frames = (xp[idx] * w[None, :]).astype(np.float32)
    spec = np.fft.rfft(frames.astype(np.float64), axis=-1)
    re, im = spec.real.astype(np.float32), spec.imag.astype(np.float32)
    mag = np.sqrt(re * re + im * im, dtype=np.float32)
    return (mag * mag).astype(np.float32)


def whisper_log_mel(samples: np.ndarray, window: np.ndarray, fbanks: np.ndarray, n_fft: int = 400, hop: int = 160,
                    n_samples: int = 480000) -> np.ndarray:
    """WhisperFeatureExtractor.extract (playground-node/src/whisper/audio.ts:322-414) for 16 kHz input:
    pad/cut to 30 s, mel power [M, T], drop the last frame, log10(max(x,1e-10)), clamp to max-8,
    (x+4)/4, with the Float32Array storage of the host loop.  Returns [1, M, 3000]."""
    x = np.zeros(n_samples, dtype=np.float32)
    s = np.asarray(samples, dtype=np.float32).reshape(-1)[:n_samples]
    x[: s.size] = s
    power = stft_power(x, window, n_fft, hop)                                  # [T, F]
    mel = linear(power, np.ascontiguousarray(np.asarray(fbanks, np.float32).T))  # [T, M], f32 accumulation as the GEMM shader
    mel = mel.T[:, : n_samples // hop]                                          # [M, 3000]
    log_spec = np.log10(np.maximum(mel.astype(np.float64), np.float64(np.float32(1e-10)))).astype(np.float32)
    mx = log_spec.max()
    log_spec = np.maximum(log_spec.astype(np.float64), np.float64(mx) - 8.0).astype(np.float32)
    return ((log_spec.astype(np.float64) + 4.0) / 4.0).astype(np.float32)[None]


def conv1d(x: np.ndarray, w: np.ndarray, bias: np.ndarray | None, stride: int = 1, padding: int = 0) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    B, Cin, L = x.shape
    Cout, Cin2, ksz = w.shape
    assert Cin == Cin2
    Wout = (L + 2 * padding - ksz) // stride + 1
    out = np.empty((B, Cout, Wout), dtype=np.float32)
    bk = _f32(bias) if bias is not None else None
    lib().orc_conv1d(_p(x), _p(w), _p(bk) if bk is not None else None, _p(out), B, Cin, L, Cout, ksz, stride, padding)
    return out


# ----------------------------------------------------------------------------- RoPE
def rope_inv_freq(dim: int, base: float) -> np.ndarray:
    """inv_freq[i] = f32(1 / base**(i/(dim/2))) computed in doubles
    (packages/model-utils/src/rope.ts:159-171)."""
    half = dim // 2
    return np.array([1.0 / math.pow(base, i / half) for i in range(half)], dtype=np.float32)


def rope_tables(positions: np.ndarray, dim: int, base: float) -> tuple[np.ndarray, np.ndarray]:
    """freqs = f32(pos) * inv_freq in fp32; emb = cat(freqs, freqs); cos/sin(emb)
    (packages/model-utils/src/rope.ts:192-261)."""
    inv = rope_inv_freq(dim, base)
    pos = positions.astype(np.float32)
    freqs = (pos[..., None] * inv).astype(np.float32)
    emb = np.concatenate([freqs, freqs], axis=-1)
    return unary("cos", emb), unary("sin", emb)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """x*cos + rotate_half(x)*sin with rotate_half(x) = cat(-x2, x1)
    (packages/model-utils/src/rope.ts:546-644).  x [B,H,S,D]; cos/sin [S,D]."""
    half = x.shape[-1] // 2
    rot = np.concatenate([-x[..., half:], x[..., :half]], axis=-1)
    return add(mul(x, cos[None, None]), mul(rot, sin[None, None]))


# ----------------------------------------------------------------------------- Qwen3
@dataclass
class Qwen3Config:
    """Field meanings follow Qwen3ModelConfig (packages/model-utils/src/qwen3/model.ts:45-84)."""
    vocab_size: int = 151936
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6


class StaticKVCacheOracle:
    """[B,Hkv,maxS,D] zero-initialised per layer; update writes [start,end) and returns the
    [:end] prefix (packages/model-utils/src/kv-cache.ts:123-130,164-212)."""

    def __init__(self, cfg: Qwen3Config, batch: int, max_seq_len: int):
        shp = (batch, cfg.num_key_value_heads, max_seq_len, cfg.head_dim)
        self.k = [np.zeros(shp, np.float32) for _ in range(cfg.num_hidden_layers)]
        self.v = [np.zeros(shp, np.float32) for _ in range(cfg.num_hidden_layers)]
        self.max_seq_len = max_seq_len

    def update(self, layer: int, k: np.ndarray, v: np.ndarray, start: int):
        end = start + k.shape[2]
        if end > self.max_seq_len:
            raise ValueError("Cache overflow")
        self.k[layer][:, :, start:end] = k
        self.v[layer][:, :, start:end] = v
        return self.k[layer][:, :, :end], self.v[layer][:, :, :end]


class Qwen3Oracle:
    """Operator sequence of Qwen3ForCausalLM.forward / forwardWithKVCache
    (packages/model-utils/src/qwen3/for_causal_lm.ts:149-194), Qwen3Model
    (qwen3/model.ts:265-347), Qwen3DecoderLayer (qwen3/decoder_layer.ts:191-241),
    GroupedQueryAttention (attention/gqa.ts:246-430) and SwiGLUMLP (mlp/swiglu.ts:119-134).

    `weights` maps HuggingFace-style names to fp32 arrays:
      model.embed_tokens.weight, model.norm.weight,
      model.layers.{i}.{input_layernorm,post_attention_layernorm}.weight,
      model.layers.{i}.self_attn.{q,k,v,o}_proj.weight, .self_attn.{q,k}_norm.weight,
      model.layers.{i}.mlp.{gate,up,down}_proj.weight.   lm_head is tied to embed_tokens.
    """

    def __init__(self, cfg: Qwen3Config, weights: dict):
        self.cfg = cfg
        self.w = weights

    def _attention(self, li: int, h: np.ndarray, cos, sin, cache, pos: int, hooks=None) -> np.ndarray:
        c, w = self.cfg, self.w
        pre = f"model.layers.{li}.self_attn."
        B, S, _ = h.shape
        q = linear(h, w[pre + "q_proj.weight"]).reshape(B, S, c.num_attention_heads, c.head_dim)
        k = linear(h, w[pre + "k_proj.weight"]).reshape(B, S, c.num_key_value_heads, c.head_dim)
        v = linear(h, w[pre + "v_proj.weight"]).reshape(B, S, c.num_key_value_heads, c.head_dim)
        q = rms_norm(q, w[pre + "q_norm.weight"], c.rms_norm_eps)      # gqa.ts:279-286
        k = rms_norm(k, w[pre + "k_norm.weight"], c.rms_norm_eps)
        q = np.ascontiguousarray(q.transpose(0, 2, 1, 3))             # gqa.ts:297-299
        k = np.ascontiguousarray(k.transpose(0, 2, 1, 3))
        v = np.ascontiguousarray(v.transpose(0, 2, 1, 3))
        q = apply_rope(q, cos, sin)                                   # gqa.ts:306-310
        k = apply_rope(k, cos, sin)
        causal = True
        if cache is not None:
            k, v = cache.update(li, k, v, pos)                        # gqa.ts:319-322
            if S == 1 and k.shape[2] > 1:
                causal = False                                        # gqa.ts:333-336
        # The reference materialises K/V repeated to Hq heads (gqa.ts:494-519) and calls the
        # kernel with ratio 1; the grouped call below reads the same rows.
        o = sdpa(q, k, v, is_causal=causal)
        if hooks is not None:
            hooks.setdefault(f"attn{li}", o)
        o = np.ascontiguousarray(o.transpose(0, 2, 1, 3)).reshape(B, S, -1)
        return linear(o, w[pre + "o_proj.weight"])

    def _mlp(self, li: int, h: np.ndarray) -> np.ndarray:
        pre = f"model.layers.{li}.mlp."
        g = unary("silu", linear(h, self.w[pre + "gate_proj.weight"]))
        u = linear(h, self.w[pre + "up_proj.weight"])
        return linear(mul(g, u), self.w[pre + "down_proj.weight"])

    def hidden(self, ids: np.ndarray, cache=None, pos: int = 0, num_layers: int | None = None, hooks=None) -> np.ndarray:
        c, w = self.cfg, self.w
        B, S = ids.shape
        h = embedding(w["model.embed_tokens.weight"], ids)
        positions = np.arange(pos, pos + S, dtype=np.int32)            # rope.ts:270-272
        cos, sin = rope_tables(positions, c.head_dim, c.rope_theta)
        L = c.num_hidden_layers if num_layers is None else num_layers
        for li in range(L):
            pre = f"model.layers.{li}."
            x = rms_norm(h, w[pre + "input_layernorm.weight"], c.rms_norm_eps)
            h = add(h, self._attention(li, x, cos, sin, cache, pos, hooks))
            x = rms_norm(h, w[pre + "post_attention_layernorm.weight"], c.rms_norm_eps)
            h = add(h, self._mlp(li, x))
            if hooks is not None:
                hooks[f"layer{li}"] = h
        return rms_norm(h, w["model.norm.weight"], c.rms_norm_eps)

    def logits(self, ids: np.ndarray, cache=None, pos: int = 0, last_only: bool = False,
               num_layers: int | None = None) -> np.ndarray:
        """Tied lm_head: matmul(h, embed^T) (for_causal_lm.ts:184-185).  The reference computes
        every position; last_only selects position S-1 before the matmul (same rows)."""
        h = self.hidden(ids, cache, pos, num_layers)
        if last_only:
            h = h[:, -1:, :]
        return linear(h, self.w["model.embed_tokens.weight"])

    def greedy_generate(self, ids: np.ndarray, steps: int, max_seq_len: int | None = None) -> np.ndarray:
        """Prefill, then `steps` greedy tokens: select last position, argmax, feed back
        (for_causal_lm.ts:475-508, batch-capable form)."""
        B, S = ids.shape
        cache = StaticKVCacheOracle(self.cfg, B, max_seq_len or (S + steps))
        out = np.empty((B, steps), dtype=np.int32)
        lg = self.logits(ids, cache, 0, last_only=True)
        tok = argmax_rows(lg[:, -1, :])
        out[:, 0] = tok
        for t in range(1, steps):
            lg = self.logits(tok.reshape(B, 1), cache, S + t - 1, last_only=True)
            tok = argmax_rows(lg[:, -1, :])
            out[:, t] = tok
        return out


# ----------------------------------------------------------------------------- Whisper encoder
@dataclass
class WhisperEncoderConfig:
    """packages/model-utils/src/whisper/config.ts:33-69 (encoder fields)."""
    n_mels: int = 80
    n_audio_ctx: int = 1500
    n_audio_state: int = 768
    n_audio_head: int = 12
    n_audio_layer: int = 12
    ln_eps: float = 1e-5


class WhisperEncoderOracle:
    """WhisperAudioEncoder.forward (packages/model-utils/src/whisper/encoder.ts:202-250) with
    ResidualAttentionBlock (whisper/block.ts:150-200) and nn.MultiheadAttention
    (packages/core/src/nn/modules/attention/MultiheadAttention.ts:280-437).

    weights: conv1.{weight,bias}, conv2.{weight,bias}, embed_positions.weight,
      layers.{i}.self_attn_layer_norm.{weight,bias}, layers.{i}.self_attn.in_proj_{weight,bias},
      layers.{i}.self_attn.out_proj.{weight,bias}, layers.{i}.final_layer_norm.{weight,bias},
      layers.{i}.fc1.{weight,bias}, layers.{i}.fc2.{weight,bias}, layer_norm.{weight,bias}
    """

    def __init__(self, cfg: WhisperEncoderConfig, weights: dict):
        self.cfg, self.w = cfg, weights

    def forward(self, mel: np.ndarray, num_layers: int | None = None) -> np.ndarray:
        c, w = self.cfg, self.w
        x = unary("gelu", conv1d(mel, w["conv1.weight"], w["conv1.bias"], 1, 1))
        x = unary("gelu", conv1d(x, w["conv2.weight"], w["conv2.bias"], 2, 1))
        x = x.transpose(0, 2, 1)                                       # [B,T,C]
        T = x.shape[1]
        x = add(x, w["embed_positions.weight"][:T][None])
        B, E, H = x.shape[0], c.n_audio_state, c.n_audio_head
        D = E // H
        L = c.n_audio_layer if num_layers is None else num_layers
        for li in range(L):
            p = f"layers.{li}."
            y = layer_norm(x, w[p + "self_attn_layer_norm.weight"], w[p + "self_attn_layer_norm.bias"], c.ln_eps)
            W_in, b_in = w[p + "self_attn.in_proj_weight"], w[p + "self_attn.in_proj_bias"]
            q = linear(y, W_in[0:E], b_in[0:E])
            k = linear(y, W_in[E:2 * E], b_in[E:2 * E])
            v = linear(y, W_in[2 * E:], b_in[2 * E:])
            def heads(t):
                return np.ascontiguousarray(t.reshape(B, T, H, D).transpose(0, 2, 1, 3)).reshape(B * H, T, D)
            o = sdpa(heads(q), heads(k), heads(v), is_causal=False)     # 3-D path: batch 1, heads B*H
            o = np.ascontiguousarray(o.reshape(B, H, T, D).transpose(0, 2, 1, 3)).reshape(B, T, E)
            x = add(x, linear(o, w[p + "self_attn.out_proj.weight"], w[p + "self_attn.out_proj.bias"]))
            y = layer_norm(x, w[p + "final_layer_norm.weight"], w[p + "final_layer_norm.bias"], c.ln_eps)
            y = unary("gelu", linear(y, w[p + "fc1.weight"], w[p + "fc1.bias"]))
            x = add(x, linear(y, w[p + "fc2.weight"], w[p + "fc2.bias"]))
        return layer_norm(x, w["layer_norm.weight"], w["layer_norm.bias"], c.ln_eps)


# ----------------------------------------------------------------------------- Whisper text decoder
@dataclass
class WhisperDecoderConfig:
    """packages/model-utils/src/whisper/config.ts (decoder fields)."""
    n_vocab: int = 51865
    n_text_ctx: int = 448
    n_text_state: int = 768
    n_text_head: int = 12
    n_text_layer: int = 12
    ln_eps: float = 1e-5


class WhisperDecoderOracle:
    """WhisperTextDecoder.forward (packages/model-utils/src/whisper/decoder.ts:203-261) with the
    cross-attention ResidualAttentionBlock (whisper/block.ts:150-200).  Self-attention carries the
    additive -inf mask, which sends scaled_dot_product_attention down the naive path
    matmul(alpha=scale) -> add(mask) -> softmax -> matmul
    (packages/core/src/dispatch/handlers/composite.ts:262-347); cross-attention has no mask and uses
    the fused attention kernel.

    weights: embed_tokens.weight, embed_positions.weight, layer_norm.{weight,bias}, and per layer
      layers.{i}.{self_attn,encoder_attn}.{in_proj_weight,in_proj_bias,out_proj.weight,out_proj.bias},
      layers.{i}.{self_attn_layer_norm,encoder_attn_layer_norm,final_layer_norm}.{weight,bias},
      layers.{i}.fc1.{weight,bias}, layers.{i}.fc2.{weight,bias}
    """

    def __init__(self, cfg: WhisperDecoderConfig, weights: dict):
        self.cfg, self.w = cfg, weights

    def _mha(self, prefix: str, xq: np.ndarray, xkv: np.ndarray, mask: np.ndarray | None) -> np.ndarray:
        c, w = self.cfg, self.w
        B, L, E = xq.shape
        S, H = xkv.shape[1], c.n_text_head
        D = E // H
        W_in, b_in = w[prefix + "in_proj_weight"], w[prefix + "in_proj_bias"]
        q = linear(xq, W_in[0:E], b_in[0:E])
        k = linear(xkv, W_in[E:2 * E], b_in[E:2 * E])
        v = linear(xkv, W_in[2 * E:], b_in[2 * E:])
        def heads(t, n):
            return np.ascontiguousarray(t.reshape(B, n, H, D).transpose(0, 2, 1, 3)).reshape(1, B * H, n, D)
        qh, kh, vh = heads(q, L), heads(k, S), heads(v, S)
        if mask is None:
            o = sdpa(qh[0], kh[0], vh[0], is_causal=False)[None]
        else:
            scores = matmul4d(qh, kh, trans_b=True, alpha=1.0 / math.sqrt(D))
            scores = add(scores, mask[None, None])
            o = matmul4d(softmax(scores), vh)
        o = np.ascontiguousarray(o.reshape(B, H, L, D).transpose(0, 2, 1, 3)).reshape(B, L, E)
        return linear(o, w[prefix + "out_proj.weight"], w[prefix + "out_proj.bias"])

    def forward(self, tokens: np.ndarray, xa: np.ndarray, offset: int = 0, num_layers: int | None = None) -> np.ndarray:
        c, w = self.cfg, self.w
        S = tokens.shape[1]
        x = add(embedding(w["embed_tokens.weight"], tokens), w["embed_positions.weight"][offset:offset + S][None])
        mask = np.where(np.arange(S)[None, :] > np.arange(S)[:, None], -np.inf, 0.0).astype(np.float32)
        L = c.n_text_layer if num_layers is None else num_layers
        for li in range(L):
            p = f"layers.{li}."
            y = layer_norm(x, w[p + "self_attn_layer_norm.weight"], w[p + "self_attn_layer_norm.bias"], c.ln_eps)
            x = add(x, self._mha(p + "self_attn.", y, y, mask))
            y = layer_norm(x, w[p + "encoder_attn_layer_norm.weight"], w[p + "encoder_attn_layer_norm.bias"], c.ln_eps)
            x = add(x, self._mha(p + "encoder_attn.", y, xa, None))
            y = layer_norm(x, w[p + "final_layer_norm.weight"], w[p + "final_layer_norm.bias"], c.ln_eps)
            y = unary("gelu", linear(y, w[p + "fc1.weight"], w[p + "fc1.bias"]))
            x = add(x, linear(y, w[p + "fc2.weight"], w[p + "fc2.bias"]))
        x = layer_norm(x, w["layer_norm.weight"], w["layer_norm.bias"], c.ln_eps)
        return linear(x, w["embed_tokens.weight"])


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
