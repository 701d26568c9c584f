"""Seeded synthetic weights and inputs for the benchmark configurations.

No real checkpoints or datasets are involved: every tensor is drawn from
numpy.random.Generator(PCG64(seed)) with a seed derived from the tensor's name, so the CPU oracle,
a single GPU and every rank of a multi-GPU run see identical values.
"""
from __future__ import annotations

import zlib

import numpy as np

BASE_SEED = 1234


def _rng(name: str, base_seed: int = BASE_SEED) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64([base_seed, zlib.crc32(name.encode())]))


def normal(name: str, shape, std: float = 1.0, mean: float = 0.0, base_seed: int = BASE_SEED) -> np.ndarray:
    a = _rng(name, base_seed).standard_normal(shape, dtype=np.float32)
    if std != 1.0:
        a *= np.float32(std)
    if mean != 0.0:
        a += np.float32(mean)
    return a


def token_ids(name: str, shape, vocab: int, base_seed: int = BASE_SEED) -> np.ndarray:
    return _rng(name, base_seed).integers(0, vocab, size=shape, dtype=np.int32)


def qwen3_weights(*, vocab: int, hidden: int, inter: int, layers: int, heads: int, kv_heads: int, head_dim: int,
                  std: float = 0.02, norm_jitter: float = 0.0, base_seed: int = BASE_SEED) -> dict:
    """HuggingFace-style names -> float32 arrays.  Linear and embedding weights ~ N(0, std);
    RMSNorm weights are ones as the modules construct them (optionally N(1, norm_jitter))."""
    w = {}

    def lin(name, out_f, in_f):
        w[name] = normal(name, (out_f, in_f), std, base_seed=base_seed)

    def nrm(name, n):
        w[name] = (normal(name, (n,), norm_jitter, 1.0, base_seed) if norm_jitter else np.ones((n,), np.float32))

    w["model.embed_tokens.weight"] = normal("model.embed_tokens.weight", (vocab, hidden), std, base_seed=base_seed)
    for i in range(layers):
        p = f"model.layers.{i}."
        lin(p + "self_attn.q_proj.weight", heads * head_dim, hidden)
        lin(p + "self_attn.k_proj.weight", kv_heads * head_dim, hidden)
        lin(p + "self_attn.v_proj.weight", kv_heads * head_dim, hidden)
        lin(p + "self_attn.o_proj.weight", hidden, heads * head_dim)
        nrm(p + "self_attn.q_norm.weight", head_dim)
        nrm(p + "self_attn.k_norm.weight", head_dim)
        lin(p + "mlp.gate_proj.weight", inter, hidden)
        lin(p + "mlp.up_proj.weight", inter, hidden)
        lin(p + "mlp.down_proj.weight", hidden, inter)
        nrm(p + "input_layernorm.weight", hidden)
        nrm(p + "post_attention_layernorm.weight", hidden)
    nrm("model.norm.weight", hidden)
    return w


def whisper_encoder_weights(*, n_mels: int, state: int, layers: int, n_ctx: int, std: float = 0.02,
                            base_seed: int = BASE_SEED) -> dict:
    w = {}

    def t(name, shape, s=std, mean=0.0):
        w[name] = normal(name, shape, s, mean, base_seed)

    t("conv1.weight", (state, n_mels, 3)); t("conv1.bias", (state,))
    t("conv2.weight", (state, state, 3)); t("conv2.bias", (state,))
    t("embed_positions.weight", (n_ctx, state))
    for i in range(layers):
        p = f"layers.{i}."
        t(p + "self_attn_layer_norm.weight", (state,), std, 1.0); t(p + "self_attn_layer_norm.bias", (state,))
        t(p + "self_attn.in_proj_weight", (3 * state, state)); t(p + "self_attn.in_proj_bias", (3 * state,))
        t(p + "self_attn.out_proj.weight", (state, state)); t(p + "self_attn.out_proj.bias", (state,))
        t(p + "final_layer_norm.weight", (state,), std, 1.0); t(p + "final_layer_norm.bias", (state,))
        t(p + "fc1.weight", (4 * state, state)); t(p + "fc1.bias", (4 * state,))
        t(p + "fc2.weight", (state, 4 * state)); t(p + "fc2.bias", (state,))
    t("layer_norm.weight", (state,), std, 1.0); t("layer_norm.bias", (state,))
    return w


def whisper_decoder_weights(*, vocab: int, state: int, layers: int, n_ctx: int, std: float = 0.02,
                            base_seed: int = BASE_SEED) -> dict:
    w = {}

    def t(name, shape, s=std, mean=0.0):
        w[name] = normal("dec." + name, shape, s, mean, base_seed)

    t("embed_tokens.weight", (vocab, state)); t("embed_positions.weight", (n_ctx, state))
    for i in range(layers):
        p = f"layers.{i}."
        for a in ("self_attn", "encoder_attn"):
            t(p + a + "_layer_norm.weight", (state,), std, 1.0); t(p + a + "_layer_norm.bias", (state,))
            t(p + a + ".in_proj_weight", (3 * state, state)); t(p + a + ".in_proj_bias", (3 * state,))
            t(p + a + ".out_proj.weight", (state, state)); t(p + a + ".out_proj.bias", (state,))
        t(p + "final_layer_norm.weight", (state,), std, 1.0); t(p + "final_layer_norm.bias", (state,))
        t(p + "fc1.weight", (4 * state, state)); t(p + "fc1.bias", (4 * state,))
        t(p + "fc2.weight", (state, 4 * state)); t(p + "fc2.bias", (state,))
    t("layer_norm.weight", (state,), std, 1.0); t("layer_norm.bias", (state,))
    return w


def synthetic_audio(name: str, n_samples: int = 480000, sr: int = 16000, base_seed: int = BASE_SEED) -> np.ndarray:
    """Sum of 3..8 sines (80..4000 Hz, amplitude 0.05..0.3, random phase) plus N(0, 0.01) noise."""
    g = _rng(name, base_seed)
    n = int(g.integers(3, 9))
    t = np.arange(n_samples, dtype=np.float64) / sr
    x = np.zeros(n_samples, dtype=np.float64)
    for _ in range(n):
        x += g.uniform(0.05, 0.3) * np.sin(2 * np.pi * g.uniform(80, 4000) * t + g.uniform(0, 2 * np.pi))
    x += g.standard_normal(n_samples) * 0.01
    return x.astype(np.float32)


class LazyQwen3Weights:
    """dict-like view of the synthetic Qwen3 weights that materialises one tensor at a time (a 4B
    model would need 16 GB of host memory per rank otherwise).  Same values as qwen3_weights().
    With `shard=(rank, world)` tensors come out as that rank's tensor-parallel slice; `transform`
    (e.g. bf16 rounding) is applied to every tensor handed out."""

    def __init__(self, *, vocab, hidden, inter, layers, heads, kv_heads, head_dim, std=0.02, norm_jitter=0.0,
                 base_seed=BASE_SEED, shard=None, transform=None):
        self.d = dict(vocab=vocab, hidden=hidden, inter=inter, layers=layers, heads=heads, kv_heads=kv_heads, head_dim=head_dim)
        self.std, self.jitter, self.seed, self.shard, self.transform = std, norm_jitter, base_seed, shard, transform

    def _shape(self, name):
        d = self.d
        if name == "model.embed_tokens.weight":
            return (d["vocab"], d["hidden"])
        if name.endswith("norm.weight"):
            return (d["head_dim"],) if ("q_norm" in name or "k_norm" in name) else (d["hidden"],)
        table = {"q_proj": (d["heads"] * d["head_dim"], d["hidden"]), "k_proj": (d["kv_heads"] * d["head_dim"], d["hidden"]),
                 "v_proj": (d["kv_heads"] * d["head_dim"], d["hidden"]), "o_proj": (d["hidden"], d["heads"] * d["head_dim"]),
                 "gate_proj": (d["inter"], d["hidden"]), "up_proj": (d["inter"], d["hidden"]), "down_proj": (d["hidden"], d["inter"])}
        for k, shp in table.items():
            if name.endswith(k + ".weight"):
                return shp
        raise KeyError(name)

    def __getitem__(self, name):
        shape = self._shape(name)
        if name.endswith("norm.weight"):
            w = normal(name, shape, self.jitter, 1.0, self.seed) if self.jitter else np.ones(shape, np.float32)
        else:
            w = normal(name, shape, self.std, base_seed=self.seed)
        if self.shard is not None and self.shard[1] > 1:
            from .parallel import shard_qwen3_weights
            w = shard_qwen3_weights({name: w}, heads=self.d["heads"], kv_heads=self.d["kv_heads"], head_dim=self.d["head_dim"],
                                    rank=self.shard[0], world=self.shard[1])[name]
        return self.transform(w) if self.transform else w
