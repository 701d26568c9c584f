"""Golden fixtures (tests/golden/oracle_golden.npz, produced by tests/golden/make_golden.py).

CPU: the oracle still reproduces its recorded outputs bit for bit on the same build flags (small
tolerance allows a different libm).  GPU: the CUDA kernels reproduce the same numbers within the
fp32 bound (1e-4 of the output's absolute maximum)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402

from kandle_b200 import synth  # noqa: E402

G = np.load(os.path.join(HERE, "golden", "oracle_golden.npz"))


def test_oracle_reproduces_golden(oracle):
    q, k, v = make_golden.config1_inputs()
    o = oracle.sdpa(q, k, v, is_causal=True)
    assert np.abs(o[:, :, ::8, :] - G["c1_sdpa_rows"]).max() <= 1e-6
    assert abs(o.astype(np.float64).sum() - G["c1_sdpa_checksum"][0]) <= 1e-3
    w, model, ids = make_golden.tiny_qwen3()
    assert np.abs(model.logits(ids) - G["tiny_logits"]).max() <= 1e-5
    assert np.array_equal(model.greedy_generate(ids, 5), G["tiny_tokens"])
    x, gw = synth.normal("golden.x", (6, 128), 2.0), synth.normal("golden.w", (128,), 0.1, 1.0)
    assert np.abs(oracle.rms_norm(x, gw, 1e-6) - G["rms_norm"]).max() <= 1e-6
    assert np.abs(oracle.layer_norm(x, gw, gw - 1.0, 1e-5) - G["layer_norm"]).max() <= 1e-6
    assert np.abs(oracle.softmax(x) - G["softmax"]).max() <= 1e-7
    assert np.abs(oracle.unary("gelu", x) - G["gelu"]).max() <= 1e-6
    cos, sin = oracle.rope_tables(np.arange(2040, 2048, dtype=np.int32), 128, 1e6)
    assert np.abs(cos - G["rope_cos"]).max() <= 1e-6 and np.abs(sin - G["rope_sin"]).max() <= 1e-6
    assert np.array_equal(make_golden.sampler_tokens(), G["sampler_tokens"])
    assert np.abs(make_golden.log_mel_golden()[1][0, ::4, ::25] - G["log_mel"]).max() <= 1e-6


@pytest.mark.gpu
def test_cuda_kernels_reproduce_golden(backend):
    from kandle_b200 import core
    from kandle_b200.core import Tensor
    from kandle_b200.model_utils import Qwen3Config, Qwen3ForCausalLM

    def close(got, ref, rel=1e-4):
        assert np.abs(got - ref).max() <= rel * np.abs(ref).max()

    q, k, v = make_golden.config1_inputs()
    o = core.scaledDotProductAttention(Tensor(q), Tensor(k), Tensor(v), None, 0.0, True).dataAsync()
    close(o[:, :, ::8, :], G["c1_sdpa_rows"])
    assert abs(o.astype(np.float64).sum() - G["c1_sdpa_checksum"][0]) <= 1e-4 * G["c1_sdpa_checksum"][1]
    w, _, ids = make_golden.tiny_qwen3()
    t = make_golden.TINY
    model = Qwen3ForCausalLM(Qwen3Config(vocabSize=t["vocab"], hiddenSize=t["hidden"], intermediateSize=t["inter"],
                                         numHiddenLayers=t["layers"], numAttentionHeads=t["heads"],
                                         numKeyValueHeads=t["kv_heads"], headDim=t["head_dim"]))
    model.loadStateDict(w)
    close(model.forward(Tensor(ids)).dataAsync(), G["tiny_logits"])
    assert np.array_equal(model.generateGreedy(Tensor(ids), 5), G["tiny_tokens"].astype(np.int64))
    x, gw = synth.normal("golden.x", (6, 128), 2.0), synth.normal("golden.w", (128,), 0.1, 1.0)
    close(core.rmsNorm(Tensor(x), (128,), Tensor(gw), 1e-6).dataAsync(), G["rms_norm"])
    close(core.layerNorm(Tensor(x), (128,), Tensor(gw), Tensor(gw - 1.0), 1e-5).dataAsync(), G["layer_norm"])
    close(core.softmax(Tensor(x)).dataAsync(), G["softmax"])
    close(core.silu(Tensor(x)).dataAsync(), G["silu"], 1e-5)
    close(core.gelu(Tensor(x)).dataAsync(), G["gelu"], 1e-5)
    from kandle_b200 import audio
    feats = audio.WhisperFeatureExtractor(80).extract(make_golden.log_mel_golden()[0], 16000).dataAsync()
    assert np.abs(feats[0, ::4, ::25] - G["log_mel"]).max() <= 1e-3
    from kandle_b200.model_utils import SamplerConfig, sample
    row, us = make_golden.sampler_inputs()
    rt = Tensor(row)
    for ci, (t_, k_, p_) in enumerate(make_golden.SAMPLER_CASES):
        got = [sample(rt, SamplerConfig(temperature=t_, topK=k_, topP=p_), uniform=float(u)).tokenId for u in us]
        assert got == list(G["sampler_tokens"][ci])
