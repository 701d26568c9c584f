"""GPU sequence tests of the Whisper audio encoder on the eager operator path (conv1d stems via
im2col + GEMM, LayerNorm, nn.MultiheadAttention with sliced in_proj weights and transposed
activations, non-causal attention with head_dim 64, tanh-GELU MLP) against the CPU oracle."""
import numpy as np
import pytest

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor
from kandle_b200.model_utils import WhisperAudioEncoder, WhisperConfig

pytestmark = pytest.mark.gpu


def _build(oracle, *, n_mels, state, heads, layers, n_ctx, dtype="float32", std=0.02):
    w = synth.whisper_encoder_weights(n_mels=n_mels, state=state, layers=layers, n_ctx=n_ctx, std=std)
    if dtype == "bfloat16":
        w = {k: lib.round_to_bf16(v) for k, v in w.items()}
    cfg = WhisperConfig(nMels=n_mels, nAudioCtx=n_ctx, nAudioState=state, nAudioHead=heads, nAudioLayer=layers, dtype=dtype)
    enc = WhisperAudioEncoder(cfg)
    enc.loadStateDict(w)
    ocfg = oracle.WhisperEncoderConfig(n_mels=n_mels, n_audio_ctx=n_ctx, n_audio_state=state, n_audio_head=heads, n_audio_layer=layers)
    return enc, oracle.WhisperEncoderOracle(ocfg, w)


def test_small_encoder_fp32(backend, oracle):
    enc, orc = _build(oracle, n_mels=8, state=32, heads=4, layers=2, n_ctx=20, std=0.1)
    names = set(enc.stateDict())
    assert "layers.1.self_attn.in_proj_weight" in names and "embed_positions.weight" in names
    mel = synth.normal("mel", (3, 8, 40))
    y = enc.forward(Tensor(mel))
    assert y.shape == (3, 20, 32)
    ref = orc.forward(mel)
    assert np.abs(y.dataAsync() - ref).max() <= 1e-4 * np.abs(ref).max()


def test_whisper_small_shapes_fp32_one_layer(backend, oracle):
    """Whisper-small shapes: 80 mel bins x 3000 frames -> 1500 x 768, 12 heads of 64."""
    enc, orc = _build(oracle, n_mels=80, state=768, heads=12, layers=1, n_ctx=1500)
    mel = synth.normal("mel", (1, 80, 3000))
    y = enc.forward(Tensor(mel)).dataAsync()
    ref = orc.forward(mel)
    assert y.shape == (1, 1500, 768)
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()


def test_whisper_small_shapes_bf16_two_layers(backend, oracle):
    """bf16 storage: the linears and the attention (S=1500, D=64, non-causal, ragged last tile) run on
    the tcgen05 kernels; every operator rounds its output to bf16 as the reference does for 16-bit
    storage, so the bound is looser than for the fused engine."""
    enc, orc = _build(oracle, n_mels=80, state=768, heads=12, layers=2, n_ctx=1500, dtype="bfloat16")
    mel = lib.round_to_bf16(synth.normal("mel", (2, 80, 3000)))
    n0 = backend.launch_count(reset=True)
    y = enc.forward(Tensor(mel, dtype="bfloat16"))
    assert y.dtype == "bfloat16"
    got = y.dataAsync()
    ref = orc.forward(mel)
    err = np.abs(got - ref)
    assert np.quantile(err, 0.999) <= 3e-2 * np.abs(ref).max() and err.max() <= 6e-2 * np.abs(ref).max(), (err.max(), np.abs(ref).max())


def _build_decoder(oracle, *, vocab, state, heads, layers, n_ctx, std=0.08):
    from kandle_b200.model_utils import WhisperTextDecoder
    w = synth.whisper_decoder_weights(vocab=vocab, state=state, layers=layers, n_ctx=n_ctx, std=std)
    cfg = WhisperConfig(nVocab=vocab, nTextCtx=n_ctx, nTextState=state, nTextHead=heads, nTextLayer=layers)
    dec = WhisperTextDecoder(cfg)
    dec.loadStateDict(w)
    ocfg = oracle.WhisperDecoderConfig(n_vocab=vocab, n_text_ctx=n_ctx, n_text_state=state, n_text_head=heads, n_text_layer=layers)
    return dec, oracle.WhisperDecoderOracle(ocfg, w)


def test_text_decoder_fp32_masked_self_attention_and_cross_attention(backend, oracle):
    """WhisperTextDecoder on the eager path: learned positions at an offset, causal self-attention
    through the additive -inf mask (the naive matmul/add/softmax/matmul path), cross-attention over
    an encoder output of a different length, logits through the transposed token embedding."""
    dec, orc = _build_decoder(oracle, vocab=203, state=64, heads=4, layers=2, n_ctx=32)
    names = set(dec.stateDict())
    assert "layers.1.encoder_attn.in_proj_weight" in names and "layers.0.encoder_attn_layer_norm.bias" in names
    tokens = synth.token_ids("dec-tokens", (2, 9), 203)
    xa = synth.normal("dec-xa", (2, 20, 64), 0.5)
    for offset in (0, 5):
        got = dec.forward(Tensor(tokens), Tensor(xa), offset).dataAsync()
        ref = orc.forward(tokens, xa, offset)
        assert got.shape == ref.shape == (2, 9, 203)
        assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()
    # causality: logits of the first 4 positions do not depend on later tokens
    t2 = tokens.copy()
    t2[:, 4:] = (t2[:, 4:] + 7) % 203
    a = dec.forward(Tensor(tokens), Tensor(xa), 0).dataAsync()
    b = dec.forward(Tensor(t2), Tensor(xa), 0).dataAsync()
    assert np.array_equal(a[:, :4], b[:, :4]) and not np.array_equal(a[:, 4:], b[:, 4:])
    with pytest.raises(ValueError):
        dec.forward(Tensor(tokens), Tensor(xa), 30)


def test_text_decoder_whisper_small_widths_one_layer(backend, oracle):
    """Whisper-small decoder widths (768 state, 12 heads of 64, vocabulary 51865) against 1500 encoder positions."""
    dec, orc = _build_decoder(oracle, vocab=51865, state=768, heads=12, layers=1, n_ctx=448, std=0.02)
    tokens = synth.token_ids("dec-tokens-small", (1, 12), 51865)
    xa = synth.normal("dec-xa-small", (1, 1500, 768), 0.3)
    got = dec.forward(Tensor(tokens), Tensor(xa)).dataAsync()
    ref = orc.forward(tokens, xa)
    assert got.shape == (1, 12, 51865)
    assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()
