"""Full-size parity runs of the benchmark configurations (slow: each builds the 0.6B model).

config 2: Qwen3-0.6B architecture, fp32, random-init N(0, 0.02), one prefill of 1 x 512 token ids,
          eager operator path (the reference's op sequence), final logits for every position.
config 3: the same architecture in bf16 on the fused engine: one sequence x 512 prompt tokens and a
          few cached decode steps against the fp32 oracle on the bf16-rounded weights; plus, at the
          benchmark's batch size, the property that sequences do not interact (a batch of identical
          prompts yields identical tokens, and equals the single-sequence run).
config 5: Whisper-small encoder, 12 layers, fp32, one 30 s clip (80 x 3000 log-mel stand-in).
"""
import numpy as np
import pytest

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor
from kandle_b200.engine import Qwen3Engine
from kandle_b200.model_utils import Qwen3Config, Qwen3ForCausalLM, WhisperAudioEncoder, WhisperConfig

pytestmark = pytest.mark.gpu
DIMS = dict(vocab=151936, hidden=1024, inter=3072, layers=28, heads=16, kv_heads=8, head_dim=128)


def _oracle_model(oracle, w):
    cfg = oracle.Qwen3Config(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                             num_attention_heads=16, num_key_value_heads=8, head_dim=128)
    return oracle.Qwen3Oracle(cfg, w)


def test_config2_qwen3_0p6b_fp32_prefill_512(backend, oracle):
    w = synth.qwen3_weights(**DIMS)
    model = Qwen3ForCausalLM(Qwen3Config())
    model.loadStateDict(w)
    ids = synth.token_ids("c2.ids", (1, 512), 151936)
    logits = model.forward(Tensor(ids))
    assert logits.shape == (1, 512, 151936)
    got = logits.dataAsync()
    ref = _oracle_model(oracle, w).logits(ids)
    err = np.abs(got - ref).max()
    assert err <= 1e-4 * np.abs(ref).max(), f"max-abs {err:.3e} vs bound {1e-4 * np.abs(ref).max():.3e}"
    assert np.array_equal(got.argmax(-1), ref.argmax(-1))


def test_config3_qwen3_0p6b_bf16_engine(backend, oracle):
    w = {k: lib.round_to_bf16(v) for k, v in synth.qwen3_weights(**DIMS).items()}
    cfg = Qwen3Config(dtype="bfloat16")
    eng = Qwen3Engine(cfg, w, 8, 640)
    ids = synth.token_ids("c3.ids", (1, 512), 151936)
    om = _oracle_model(oracle, w)
    tok, logits = eng.prefill(ids, all_logits=True)
    ref = om.logits(ids)
    got = logits.dataAsync()
    err = np.abs(got - ref)
    assert np.quantile(err, 0.999) <= 2e-2 and err.max() <= 3.5e-2, (err.max(), np.quantile(err, 0.999))
    # With random-init weights the 151 936 logits of a position are nearly flat: the oracle's own
    # top-2 gap is below the 2e-2 logit tolerance on ~15 % of positions, where bf16 cannot decide the
    # argmax.  Measured: 97.7 % identical over all positions, 100 % where the gap exceeds 2e-2.
    same = got.reshape(-1, 151936).argmax(-1) == ref.reshape(-1, 151936).argmax(-1)
    top2 = np.partition(ref.reshape(-1, 151936), -2, axis=-1)[:, -2:]
    decidable = (top2[:, 1] - top2[:, 0]) > 2e-2
    assert same[decidable].mean() >= 0.995 and same.mean() >= 0.95, (same[decidable].mean(), same.mean(), decidable.mean())
    steps = 8
    toks = eng.generate(ids, steps)
    seq = np.concatenate([ids, toks[:, :-1].astype(np.int32)], axis=1)
    picks = om.logits(seq)[:, 511:].argmax(-1)          # teacher-forced on the engine's own tokens
    assert (picks == toks).mean() >= 0.75, (picks, toks)
    # independence of sequences at batch 8: identical prompts -> identical rows == the single-sequence run
    t8 = eng.generate(np.repeat(ids, 8, axis=0), steps)
    assert (t8 == t8[0]).all() and np.array_equal(t8[:1], toks)
    eng.dispose()


def test_config5_whisper_small_encoder_fp32_12_layers(backend, oracle):
    w = synth.whisper_encoder_weights(n_mels=80, state=768, layers=12, n_ctx=1500)
    enc = WhisperAudioEncoder(WhisperConfig())
    enc.loadStateDict(w)
    mel = synth.normal("c5.mel", (1, 80, 3000), 0.5)
    y = enc.forward(Tensor(mel)).dataAsync()
    ocfg = oracle.WhisperEncoderConfig()
    ref = oracle.WhisperEncoderOracle(ocfg, w).forward(mel)
    assert y.shape == (1, 1500, 768)
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()
