"""Per-kernel micro-benchmarks through the C ABI, timed with CUDA events on the library's stream.

    python -m kandle_b200.microbench gemm  --m 65536 --n 4096 --k 1024 [--epilogue none|residual|swiglu]
    python -m kandle_b200.microbench attn  --b 4 --hq 16 --hkv 8 --s 2048 --d 128 [--no-causal]
    python -m kandle_b200.microbench decode_attn --b 32 --hq 16 --hkv 8 --ctx 2176 --d 128
    python -m kandle_b200.microbench skinny --m 32 --n 151936 --k 1024
    python -m kandle_b200.microbench chain --m 32 --hidden 1024 --attn 2048 --inter 3072 --qkv 4096
    python -m kandle_b200.microbench layer --m 32 --hidden 1024 --attn 2048 --inter 3072 --hq 16 --hkv 8
    python -m kandle_b200.microbench whisper_encoder --clips 64 [--eager]

Each run prints one JSON line with the average launch time, the algorithmic work per launch and
the achieved rate.  Inputs are seeded normal values (constant fills would flatter the power
draw); every working set used here is larger than L2 or is rewritten between iterations by the
kernel's own output.
"""
from __future__ import annotations

import argparse
import ctypes
import json

import numpy as np

import kandle_b200
from kandle_b200 import core, lib
from kandle_b200.backend import CudaEvent
from kandle_b200.core import Tensor


def _rand_bf16(shape, seed: int, std: float = 1.0) -> Tensor:
    rng = np.random.Generator(np.random.PCG64(seed))
    n = int(np.prod(shape))
    # generate a 4 Mi-element block and tile it: host RNG time stays bounded for GB-sized tensors
    blk = (rng.standard_normal(min(n, 1 << 22), dtype=np.float32) * np.float32(std))
    a = np.resize(blk, n).reshape(shape)
    return Tensor(a, dtype="bfloat16")


def _time(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    e0, e1 = CudaEvent(), CudaEvent()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    return e0.elapsed_ms(e1) / iters


def bench_gemm(a) -> dict:
    epi = {"none": 0, "residual": 1, "swiglu": 2}[a.epilogue]
    x, w = _rand_bf16((a.m, a.k), 1), _rand_bf16((a.n, a.k), 2, 0.02)
    n_out = a.n // 2 if epi == 2 else a.n
    out = core.empty((a.m, n_out), "bfloat16")
    r = _rand_bf16((a.m, a.n), 3) if epi == 1 else None
    args = (ctypes.byref(x._handle.c()), ctypes.byref(w._handle.c()), ctypes.byref(r._handle.c()) if r else None, epi,
            ctypes.byref(out._handle.c()))
    ms = _time(lambda: lib.call("kd_linear_bf16", *args), a.iters, a.warmup)
    flops = 2.0 * a.m * a.n * a.k
    return {"kernel": "gemm_bf16_tcgen05", "m": a.m, "n": a.n, "k": a.k, "epilogue": a.epilogue, "us": ms * 1e3,
            "flops": flops, "tflops": flops / ms / 1e9}


def bench_attn(a) -> dict:
    causal = not a.no_causal
    q, k, v = _rand_bf16((a.b, a.hq, a.s, a.d), 1), _rand_bf16((a.b, a.hkv, a.s, a.d), 2), _rand_bf16((a.b, a.hkv, a.s, a.d), 3)
    out = core.empty((a.b, a.hq, a.s, a.d), "bfloat16")
    scale = 1.0 / float(np.sqrt(a.d))
    args = (ctypes.byref(q._handle.c()), ctypes.byref(k._handle.c()), ctypes.byref(v._handle.c()),
            ctypes.byref(out._handle.c()), ctypes.c_float(scale), int(causal))
    ms = _time(lambda: lib.call("kd_flash_attention", *args), a.iters, a.warmup)
    pairs = a.s * (a.s + 1) / 2 if causal else a.s * a.s
    flops = 4.0 * a.b * a.hq * a.d * pairs
    return {"kernel": "flash_attention_tcgen05", "b": a.b, "hq": a.hq, "hkv": a.hkv, "s": a.s, "d": a.d, "causal": causal,
            "us": ms * 1e3, "flops": flops, "tflops": flops / ms / 1e9}


def bench_decode_attn(a) -> dict:
    max_s = (a.ctx + 127) // 128 * 128
    q = _rand_bf16((a.b, a.hq, 1, a.d), 1)
    # several cache slabs visited round-robin so that every launch streams from HBM, not from L2
    slabs = [(_rand_bf16((a.b, a.hkv, max_s, a.d), 10 + i), _rand_bf16((a.b, a.hkv, max_s, a.d), 20 + i)) for i in range(a.slabs)]
    out = core.empty((a.b, a.hq, 1, a.d), "bfloat16")
    scale = ctypes.c_float(1.0 / float(np.sqrt(a.d)))
    state = {"i": 0}

    def run():
        k, v = slabs[state["i"] % a.slabs]
        state["i"] += 1
        lib.call("kd_attention_decode", ctypes.byref(q._handle.c()), ctypes.byref(k._handle.c()), ctypes.byref(v._handle.c()), None,
                 a.ctx, scale, a.splits, ctypes.byref(out._handle.c()))
    ms = _time(run, a.iters, a.warmup)
    nbytes = 2.0 * a.b * a.hkv * a.ctx * a.d * 2
    return {"kernel": "flash_attention_tcgen05<decode>+combine", "b": a.b, "hq": a.hq, "hkv": a.hkv, "ctx": a.ctx, "d": a.d,
            "splits": a.splits, "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6}


def bench_skinny(a) -> dict:
    x, w = _rand_bf16((a.m, a.k), 1), _rand_bf16((a.n, a.k), 2, 0.02)
    out = core.empty((a.m, a.n), "bfloat16")
    args = (ctypes.byref(x._handle.c()), ctypes.byref(w._handle.c()), 0, ctypes.byref(out._handle.c()))
    ms = _time(lambda: lib.call("kd_linear_bf16_skinny", *args), a.iters, a.warmup)
    nbytes = 2.0 * a.n * a.k
    return {"kernel": "gemm_skinny_tcgen05", "m": a.m, "n": a.n, "k": a.k, "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6}


def bench_chain(a) -> dict:
    """kd_decode_layer_chain over several weight sets visited round-robin, so that every launch
    streams its weights from HBM as a decode step does (one layer's weights are ~30 MB, L2 is 126 MB)."""
    m, H, Ko, I, Nq = a.m, a.hidden, a.attn, a.inter, a.qkv
    sets = []
    for i in range(a.sets):
        sets.append({"wo": _rand_bf16((H, Ko), 10 + i, 0.03), "wgu": _rand_bf16((2 * I, H), 20 + i, 0.03),
                     "wd": _rand_bf16((H, I), 30 + i, 0.03), "wq": _rand_bf16((Nq, H), 40 + i, 0.03)})
    attn = _rand_bf16((m, Ko), 1)
    post, nxt = _rand_bf16((H,), 2), _rand_bf16((H,), 3)
    h = Tensor(np.zeros((m, H), np.float32))
    h1, h2 = core.empty((m, H), "float32"), core.empty((m, H), "float32")
    x, act = core.empty((m, H), "bfloat16"), core.empty((m, I), "bfloat16")
    sp = ctypes.c_int(0)
    lib.call("kd_decode_layer_chain_splits", ctypes.c_int64(Nq), ctypes.c_int64(H), ctypes.byref(sp))
    qp = core.empty((sp.value, m, Nq), "float32")
    r = lambda t: ctypes.byref(t._handle.c())  # noqa: E731
    state = {"i": 0}

    def run():
        w = sets[state["i"] % a.sets]
        state["i"] += 1
        lib.call("kd_decode_layer_chain", r(attn), r(w["wo"]), r(h), r(post), r(w["wgu"]), r(w["wd"]), r(nxt),
                 ctypes.c_float(1e-6), r(w["wq"]), r(h1), r(h2), r(x), r(act), r(qp))
    ms = _time(run, a.iters, a.warmup)
    nbytes = 2.0 * (H * Ko + 2 * I * H + H * I + Nq * H)
    return {"kernel": "decode_chain_kernel", "m": m, "hidden": H, "attn": Ko, "inter": I, "qkv": Nq, "weight_sets": a.sets,
            "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6}


def bench_layer(a) -> dict:
    """kd_decode_layer_fused over several weight sets visited round-robin (see bench_chain)."""
    m, H, Ko, I, hq, hkv = a.m, a.hidden, a.attn, a.inter, a.hq, a.hkv
    Nq = (hq + 2 * hkv) * 128
    sets = []
    for i in range(a.sets):
        sets.append({"wo": _rand_bf16((H, Ko), 10 + i, 0.03), "wgu": _rand_bf16((2 * I, H), 20 + i, 0.03),
                     "wd": _rand_bf16((H, I), 30 + i, 0.03), "wq": _rand_bf16((Nq, H), 40 + i, 0.03),
                     "kc": core.zeros((m, hkv, 64, 128), "bfloat16"), "vc": core.zeros((m, hkv, 64, 128), "bfloat16")})
    attn = _rand_bf16((m, Ko), 1)
    post, nxt, qw, kw = _rand_bf16((H,), 2), _rand_bf16((H,), 3), _rand_bf16((128,), 4), _rand_bf16((128,), 5)
    h = Tensor(np.zeros((m, H), np.float32))
    h2 = core.empty((m, H), "float32")
    cos, sin = Tensor(np.ones((1, 64), np.float32)), Tensor(np.zeros((1, 64), np.float32))
    pos = Tensor(np.array([3], np.int32))
    q = core.empty((m, 1, hq, 128), "bfloat16")
    r = lambda t: ctypes.byref(t._handle.c())  # noqa: E731
    state = {"i": 0}

    def run():
        w = sets[state["i"] % a.sets]
        state["i"] += 1
        lib.call("kd_decode_layer_fused", r(attn), r(w["wo"]), r(h), r(post), r(w["wgu"]), r(w["wd"]), r(nxt), ctypes.c_float(1e-6),
                 r(w["wq"]), r(qw), r(kw), r(cos), r(sin), r(pos), r(w["kc"]), r(w["vc"]), None, r(q), r(h2), None)
    ms = _time(run, a.iters, a.warmup)
    nbytes = 2.0 * (H * Ko + 2 * I * H + H * I + Nq * H)
    import os
    if os.environ.get("KD_DECODE_LAYER_TRACE") == "1":
        # phase timeline of the last launch: for each phase, when the first / last CTA saw its
        # dependency, had its accumulator, had published (microseconds after the earliest CTA start)
        buf = (ctypes.c_uint64 * (148 * 16))()
        lib.call("kd_debug_decode_layer_trace", buf, 148 * 16)
        t = np.array(buf, dtype=np.float64).reshape(-1, 16)
        t0 = t[:, 0][t[:, 0] > 0].min()
        rows = []
        for g in range(4):
            row = {}
            for name, col in (("dep_seen", 1 + 3 * g), ("acc_ready", 2 + 3 * g), ("published", 3 + 3 * g)):
                v = t[:, col][t[:, col] > 0]
                row[name] = [round(float(v.min() - t0) / 1e3, 2), round(float(v.max() - t0) / 1e3, 2), int(v.size)] if v.size else None
            rows.append(row)
        print(json.dumps({"trace_us_first_last_count": rows, "start_spread_us": round(float(t[:, 0].max() - t0) / 1e3, 2)}))
    return {"kernel": "decode_layer_kernel", "m": m, "hidden": H, "attn": Ko, "inter": I, "qkv": Nq, "weight_sets": a.sets,
            "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6}


def bench_whisper_encoder(a) -> dict:
    """Whisper-small audio encoder (80 mel bins x 3000 frames -> 1500 x 768, 12 layers, 12 heads of
    64) over a batch of clips in bf16 with seeded random weights: the fused fast path
    (kandle_b200/whisper_engine.py), or with --eager the operator-by-operator module.
    Algorithmic work: 344.2 GFLOP per clip (conv stems 6.4, per layer 21.2 linear + 6.9 attention)."""
    from kandle_b200 import synth
    from kandle_b200.model_utils import WhisperAudioEncoder, WhisperConfig
    from kandle_b200.whisper_engine import WhisperEncoderEngine
    w = synth.whisper_encoder_weights(n_mels=80, state=768, layers=a.layers, n_ctx=1500, std=0.02)
    w = {k: lib.round_to_bf16(v) for k, v in w.items()}
    cfg = WhisperConfig(nMels=80, nAudioCtx=1500, nAudioState=768, nAudioHead=12, nAudioLayer=a.layers, dtype="bfloat16")
    enc = WhisperAudioEncoder(cfg)
    enc.loadStateDict(w)
    mel = _rand_bf16((a.clips, 80, 3000), 7)
    run_enc = enc if a.eager else WhisperEncoderEngine(enc)

    def run():
        run_enc.forward(mel).dispose()
    ms = _time(run, a.iters, a.warmup)
    flops = a.clips * (6.4e9 + a.layers * 28.15e9)
    return {"kernel": "whisper_encoder_" + ("eager" if a.eager else "engine"), "clips": a.clips, "layers": a.layers, "ms": ms,
            "clips_per_s": a.clips / ms * 1e3, "flops": flops, "tflops": flops / ms / 1e9}


def main() -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="which", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=65536)
    g.add_argument("--n", type=int, default=4096)
    g.add_argument("--k", type=int, default=1024)
    g.add_argument("--epilogue", default="none", choices=["none", "residual", "swiglu"])
    t = sub.add_parser("attn")
    t.add_argument("--b", type=int, default=4)
    t.add_argument("--hq", type=int, default=16)
    t.add_argument("--hkv", type=int, default=8)
    t.add_argument("--s", type=int, default=2048)
    t.add_argument("--d", type=int, default=128)
    t.add_argument("--no-causal", action="store_true")
    dd = sub.add_parser("decode_attn")
    dd.add_argument("--b", type=int, default=32)
    dd.add_argument("--hq", type=int, default=16)
    dd.add_argument("--hkv", type=int, default=8)
    dd.add_argument("--ctx", type=int, default=2176)
    dd.add_argument("--d", type=int, default=128)
    dd.add_argument("--splits", type=int, default=0)
    dd.add_argument("--slabs", type=int, default=3)
    sk = sub.add_parser("skinny")
    sk.add_argument("--m", type=int, default=32)
    sk.add_argument("--n", type=int, default=151936)
    sk.add_argument("--k", type=int, default=1024)
    ch = sub.add_parser("chain")
    ch.add_argument("--m", type=int, default=32)
    ch.add_argument("--hidden", type=int, default=1024)
    ch.add_argument("--attn", type=int, default=2048)
    ch.add_argument("--inter", type=int, default=3072)
    ch.add_argument("--qkv", type=int, default=4096)
    ch.add_argument("--sets", type=int, default=8)
    ly = sub.add_parser("layer")
    ly.add_argument("--m", type=int, default=32)
    ly.add_argument("--hidden", type=int, default=1024)
    ly.add_argument("--attn", type=int, default=2048)
    ly.add_argument("--inter", type=int, default=3072)
    ly.add_argument("--hq", type=int, default=16)
    ly.add_argument("--hkv", type=int, default=8)
    ly.add_argument("--sets", type=int, default=8)
    we = sub.add_parser("whisper_encoder")
    we.add_argument("--clips", type=int, default=64)
    we.add_argument("--layers", type=int, default=12)
    we.add_argument("--eager", action="store_true")
    for p in (g, t, dd, sk, ch, ly, we):
        p.add_argument("--iters", type=int, default=10)
        p.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    kandle_b200.init(0)
    res = {"gemm": bench_gemm, "attn": bench_attn, "decode_attn": bench_decode_attn, "skinny": bench_skinny,
           "chain": bench_chain, "layer": bench_layer, "whisper_encoder": bench_whisper_encoder}[a.which](a)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
