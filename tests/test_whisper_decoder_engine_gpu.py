"""The Whisper text decoder's bf16 fast path (self-attention KV cache, encoder keys / values
projected once per clip, bias / GELU / residual in the GEMM epilogues, split-KV decode attention
for the single-position steps) against the fp32 oracle of the reference's decoder forward
(packages/model-utils/src/whisper/decoder.ts:203-261), which recomputes every position at every
step: the logits of position t from a cached step must equal the logits of position t from the
oracle's full forward over tokens[:t+1].  bf16 bound as for the encoder fast path: 99.9 % of the
logits within 2e-2 of the largest |logit|, all within 5e-2."""
import numpy as np
import pytest

from kandle_b200 import lib, synth
from kandle_b200.core import Tensor
from kandle_b200.model_utils import WhisperConfig, WhisperTextDecoder
from kandle_b200.whisper_decoder_engine import WhisperDecoderEngine

pytestmark = pytest.mark.gpu


def _build(oracle, *, vocab, state, heads, layers, n_ctx, std):
    w = {k: lib.round_to_bf16(v) for k, v in synth.whisper_decoder_weights(vocab=vocab, state=state, layers=layers, n_ctx=n_ctx, std=std).items()}
    cfg = WhisperConfig(nVocab=vocab, nTextCtx=n_ctx, nTextState=state, nTextHead=heads, nTextLayer=layers, dtype="bfloat16")
    dec = WhisperTextDecoder(cfg)
    dec.loadStateDict(w)
    ocfg = oracle.WhisperDecoderConfig(n_vocab=vocab, n_text_ctx=n_ctx, n_text_state=state, n_text_head=heads, n_text_layer=layers)
    return dec, oracle.WhisperDecoderOracle(ocfg, w)


def _check(got, ref, what):
    err = np.abs(got.astype(np.float64) - ref)
    scale = np.abs(ref).max()
    assert np.quantile(err, 0.999) <= 2e-2 * scale and err.max() <= 5e-2 * scale, (what, np.quantile(err, 0.999) / scale, err.max() / scale)


def test_cached_steps_equal_the_oracles_full_forward(backend, oracle):
    dec, orc = _build(oracle, vocab=300, state=128, heads=2, layers=3, n_ctx=40, std=0.06)
    eng = WhisperDecoderEngine(dec, 3)
    xa = lib.round_to_bf16(synth.normal("wd.xa", (3, 70, 128), 0.5))
    tokens = synth.token_ids("wd.tokens", (3, 12), 300)
    eng.set_audio(Tensor(xa, dtype="bfloat16"))
    # the prompt: 5 positions at once, logits for all of them
    got = eng.forward(tokens[:, :5], all_logits=True).dataAsync()
    ref = orc.forward(tokens, xa)                         # [3, 12, 300], every position from the full forward
    assert got.shape == (3, 5, 300)
    _check(got, ref[:, :5], "prompt")
    # single-position steps on the cache (teacher-forced tokens)
    for t in range(5, 12):
        step = eng.step(tokens[:, t]).dataAsync()
        assert step.shape == (3, 1, 300)
        _check(step[:, 0], ref[:, t], f"step at position {t}")
    # a new clip resets the text position; fewer clips than the engine's capacity
    eng.set_audio(Tensor(xa[:2], dtype="bfloat16"))
    _check(eng.forward(tokens[:2, :4]).dataAsync()[:, 0], ref[:2, 3], "second clip")
    with pytest.raises(ValueError):
        eng.forward(tokens[:2, :3])                       # several positions after the start
    with pytest.raises(ValueError):
        eng.step(tokens[:3, 0])                           # three rows for two clips
    # greedy generation: the engine's tokens against a teacher-forced oracle re-forward
    eng.set_audio(Tensor(xa, dtype="bfloat16"))
    gen = eng.generate_greedy(tokens[:, :4], 6)
    seq = np.concatenate([tokens[:, :4], gen[:, :-1].astype(np.int32)], axis=1)
    picks = orc.forward(seq, xa)[:, 3:].argmax(-1)
    assert (picks == gen).mean() >= 0.8, (picks, gen)
    eng.dispose()


def test_whisper_small_widths_against_1500_encoder_frames(backend, oracle):
    """768 state, 12 heads of 64, vocabulary 51865, two layers; 1500 encoder positions (a ragged last
    key tile in the cross attention), prompt of four tokens and three cached steps."""
    dec, orc = _build(oracle, vocab=51865, state=768, heads=12, layers=2, n_ctx=448, std=0.02)
    eng = WhisperDecoderEngine(dec, 2)
    xa = lib.round_to_bf16(synth.normal("wd.xa.small", (2, 1500, 768), 0.3))
    tokens = synth.token_ids("wd.tokens.small", (2, 7), 51865)
    eng.set_audio(Tensor(xa, dtype="bfloat16"))
    ref = orc.forward(tokens, xa)
    _check(eng.forward(tokens[:, :4]).dataAsync()[:, 0], ref[:, 3], "prompt")
    for t in range(4, 7):
        _check(eng.step(tokens[:, t]).dataAsync()[:, 0], ref[:, t], f"step at position {t}")
    eng.dispose()


def test_engine_rejects_fp32_decoders(backend):
    cfg = WhisperConfig(nVocab=50, nTextCtx=16, nTextState=128, nTextHead=2, nTextLayer=1)
    with pytest.raises(ValueError):
        WhisperDecoderEngine(WhisperTextDecoder(cfg), 1)
