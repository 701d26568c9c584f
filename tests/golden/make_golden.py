"""Generates the golden fixtures in this directory from the CPU oracle.

The reference (final-kk/kandle) ships no golden vectors for this path and cannot be executed here
(WebGPU only, no JS runtime), so these fixtures pin the ORACLE'S OWN outputs on seeded inputs: the
CPU suite checks that the oracle still reproduces them (guards against drift of the restatement),
the GPU suite checks the CUDA kernels against the same numbers.  Inputs are regenerated from their
seeds by kandle_b200.synth, so only outputs are stored.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from kandle_b200 import synth  # noqa: E402
from oracle import oracle as orc  # noqa: E402

TINY = dict(vocab=97, hidden=64, inter=96, layers=2, heads=4, kv_heads=2, head_dim=32)


def config1_inputs():
    return (synth.normal("c1.q", (1, 16, 128, 128)), synth.normal("c1.k", (1, 8, 128, 128)), synth.normal("c1.v", (1, 8, 128, 128)))


def tiny_qwen3():
    w = synth.qwen3_weights(std=0.1, norm_jitter=0.05, **TINY)
    cfg = orc.Qwen3Config(vocab_size=97, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=32)
    return w, orc.Qwen3Oracle(cfg, w), synth.token_ids("golden.ids", (2, 11), 97)


SAMPLER_CASES = [(1.0, 0, 1.0), (0.7, 50, 1.0), (1.0, 0, 0.9), (0.8, 40, 0.95), (1.3, 5, 0.5)]


def sampler_inputs():
    row = synth.normal("golden.sample", (4099,), 2.5)
    us = ((np.arange(16) + 0.5) / 16).astype(np.float32)
    return row, us


def sampler_tokens():
    row, us = sampler_inputs()
    return np.array([[orc.sample(row, t, k, p, True, float(u))["token"] for u in us] for t, k, p in SAMPLER_CASES], dtype=np.int64)


def log_mel_golden():
    from kandle_b200 import audio
    x = synth.synthetic_audio("golden.audio", 16000 * 4)
    full = orc.whisper_log_mel(x, audio.hann_window_host(400), audio.melscale_fbanks_host(201, 0, 8000, 80, 16000, "slaney", "slaney"))
    return x, full


def main():
    orc.build()
    q, k, v = config1_inputs()
    o = orc.sdpa(q, k, v, is_causal=True)
    w, model, ids = tiny_qwen3()
    x = synth.normal("golden.x", (6, 128), 2.0)
    gw = synth.normal("golden.w", (128,), 0.1, 1.0)
    cos, sin = orc.rope_tables(np.arange(2040, 2048, dtype=np.int32), 128, 1e6)
    np.savez_compressed(
        os.path.join(HERE, "oracle_golden.npz"),
        c1_sdpa_rows=o[:, :, ::8, :].astype(np.float32),                      # every 8th query row of config 1
        c1_sdpa_checksum=np.array([o.astype(np.float64).sum(), np.abs(o).astype(np.float64).sum()]),
        tiny_logits=model.logits(ids),
        tiny_tokens=model.greedy_generate(ids, 5),
        rms_norm=orc.rms_norm(x, gw, 1e-6),
        layer_norm=orc.layer_norm(x, gw, gw - 1.0, 1e-5),
        softmax=orc.softmax(x),
        silu=orc.unary("silu", x), gelu=orc.unary("gelu", x),
        rope_cos=cos, rope_sin=sin,
        sampler_tokens=sampler_tokens(),
        log_mel=log_mel_golden()[1][0, ::4, ::25],          # every 4th mel band, every 25th frame of a 4 s clip
    )
    print("wrote", os.path.join(HERE, "oracle_golden.npz"))


if __name__ == "__main__":
    main()
