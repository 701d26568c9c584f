"""GPU parity of the bf16 Whisper-encoder fast path (kandle_b200/whisper_engine.py) and of the GEMM
epilogue it is built on (kd_linear_bf16_bias: bias, tanh-form GELU, residual) against the CPU oracle
(packages/model-utils/src/whisper/encoder.ts:202-250, block.ts:150-200) and against the eager
operator path of the same encoder."""
import ctypes

import numpy as np
import pytest

from kandle_b200 import core, lib, synth
from kandle_b200.core import Tensor
from kandle_b200.model_utils import WhisperAudioEncoder, WhisperConfig
from kandle_b200.whisper_engine import WhisperEncoderEngine

pytestmark = pytest.mark.gpu


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


def _rb(a):
    return lib.round_to_bf16(np.ascontiguousarray(a, dtype=np.float32))


@pytest.mark.parametrize("M,N,K,bias,act,resid", [
    (300, 768, 768, True, 0, True),        # out_proj / fc2 form, ragged last row tile
    (257, 3072, 768, True, 1, False),      # fc1 form: bias + GELU
    (128, 2304, 768, True, 0, False),      # packed in_proj
    (64, 96, 64, False, 1, True),          # narrow tile kernel, no bias
    (1500, 72, 256, True, 1, True),        # N not a multiple of the tile width
])
def test_linear_bias_gelu_residual_epilogue(backend, oracle, M, N, K, bias, act, resid):
    x = _rb(synth.normal(f"lb-x{M}", (M, K)))
    w = _rb(synth.normal(f"lb-w{N}", (N, K), 0.05))
    b = _rb(synth.normal(f"lb-b{N}", (N,), 0.5)) if bias else None
    r = _rb(synth.normal(f"lb-r{M}", (M, N))) if resid else None
    ref = oracle.linear(x, w)
    if b is not None:
        ref = ref + b[None, :]
    if act:
        ref = oracle.unary("gelu", ref.astype(np.float32))
    if r is not None:
        ref = ref + r
    bf = lambda a: Tensor(a, dtype="bfloat16") if a is not None else None  # noqa: E731
    tx, tw, tb, tr = bf(x), bf(w), bf(b), bf(r)
    out = core.empty((M, N), "bfloat16")
    lib.call("kd_linear_bf16_bias", _r(tx), _r(tw), _r(tb), _r(tr), act, _r(out))
    got = out.dataAsync()
    # one bf16 rounding of the result (2^-9 relative) plus fp32 accumulation-order noise
    err = np.abs(got.astype(np.float64) - ref)
    assert (err <= np.abs(ref) * 2.0 ** -8 + 1e-5 * np.abs(ref).max()).all(), err.max()


def test_linear_bias_takes_a_row_slice_of_a_packed_weight_and_rejects_bad_operands(backend, oracle):
    E = 128
    x = _rb(synth.normal("lbs-x", (200, E)))
    wp = _rb(synth.normal("lbs-w", (3 * E, E), 0.05))
    bp = _rb(synth.normal("lbs-b", (3 * E,), 0.5))
    tx, tw, tb = Tensor(x, dtype="bfloat16"), Tensor(wp, dtype="bfloat16"), Tensor(bp, dtype="bfloat16")
    w1 = tw.slice([slice(E, 2 * E), slice(None)])         # the k rows, a view with a non-zero offset
    b1 = tb.slice([slice(E, 2 * E)])
    out = core.empty((200, E), "bfloat16")
    lib.call("kd_linear_bf16_bias", _r(tx), _r(w1), _r(b1), None, 0, _r(out))
    ref = oracle.linear(x, wp[E:2 * E]) + bp[None, E:2 * E]
    err = np.abs(out.dataAsync().astype(np.float64) - ref)
    assert (err <= np.abs(ref) * 2.0 ** -8 + 1e-5 * np.abs(ref).max()).all()
    with pytest.raises(lib.KandleCudaError):              # fp32 output is not part of this entry point
        lib.call("kd_linear_bf16_bias", _r(tx), _r(w1), _r(b1), None, 0, _r(core.empty((200, E), "float32")))
    with pytest.raises(lib.KandleCudaError):              # bias of the wrong length
        lib.call("kd_linear_bf16_bias", _r(tx), _r(w1), _r(tb), None, 0, _r(out))
    with pytest.raises(lib.KandleCudaError):              # unknown activation
        lib.call("kd_linear_bf16_bias", _r(tx), _r(w1), _r(b1), None, 7, _r(out))


@pytest.mark.parametrize("B,Cin,L,Cout,ksz,stride,pad,act,resid", [
    (2, 80, 300, 768, 3, 1, 1, 1, False),      # Whisper conv1 form (bias + GELU)
    (3, 64, 101, 96, 3, 2, 1, 1, True),        # conv2 form: stride 2, odd length, position residual
    (1, 8, 16, 8, 1, 1, 0, 0, False),          # pointwise conv, one clip, narrow GEMM tile
    (2, 16, 37, 40, 5, 3, 2, 0, True),         # wider kernel, stride 3, padding 2
])
def test_conv1d_tokens_against_the_channel_first_oracle(backend, oracle, B, Cin, L, Cout, ksz, stride, pad, act, resid):
    """kd_conv1d_tokens_bf16 = the reference's conv1d (im2col.ts:124-268) on a permuted layout: feed the
    oracle the channel-first tensors, compare with its output permuted to (0,2,1)."""
    x = _rb(synth.normal(f"ct-x{Cin}", (B, Cin, L)))
    w = _rb(synth.normal(f"ct-w{Cout}", (Cout, Cin, ksz), 0.1))
    b = _rb(synth.normal(f"ct-b{Cout}", (Cout,), 0.5))
    ref = oracle.conv1d(x, w, b, stride, pad)                     # [B, Cout, Wout]
    Wout = ref.shape[2]
    if act:
        ref = oracle.unary("gelu", ref)
    ref = np.ascontiguousarray(ref.transpose(0, 2, 1))
    r = _rb(synth.normal(f"ct-r{Cout}", (B, Wout, Cout))) if resid else None
    if r is not None:
        ref = ref + r
    bf = lambda a: Tensor(np.ascontiguousarray(a), dtype="bfloat16") if a is not None else None  # noqa: E731
    tx = bf(x.transpose(0, 2, 1))                                 # [B, L, Cin]
    tw = bf(w.transpose(0, 2, 1).reshape(Cout, ksz * Cin))        # tap index in front of the channel index
    tb, tr = bf(b), bf(r)
    out = core.empty((B, Wout, Cout), "bfloat16")
    lib.call("kd_conv1d_tokens_bf16", _r(tx), _r(tw), _r(tb), _r(tr), act, ksz, stride, pad, _r(out))
    err = np.abs(out.dataAsync().astype(np.float64) - ref)
    assert (err <= np.abs(ref) * 2.0 ** -8 + 1e-5 * np.abs(ref).max()).all(), err.max()
    with pytest.raises(lib.KandleCudaError):                      # weight of the wrong width
        lib.call("kd_conv1d_tokens_bf16", _r(tx), _r(tw), _r(tb), None, act, ksz + 1, stride, pad, _r(out))


def _build(oracle, *, n_mels, state, heads, layers, n_ctx, std):
    w = synth.whisper_encoder_weights(n_mels=n_mels, state=state, layers=layers, n_ctx=n_ctx, std=std)
    w = {k: lib.round_to_bf16(v) for k, v in w.items()}
    cfg = WhisperConfig(nMels=n_mels, nAudioCtx=n_ctx, nAudioState=state, nAudioHead=heads, nAudioLayer=layers, dtype="bfloat16")
    enc = WhisperAudioEncoder(cfg)
    enc.loadStateDict(w)
    ocfg = oracle.WhisperEncoderConfig(n_mels=n_mels, n_audio_ctx=n_ctx, n_audio_state=state, n_audio_head=heads, n_audio_layer=layers)
    return enc, oracle.WhisperEncoderOracle(ocfg, w)


def _check(got, ref, q999, worst):
    err = np.abs(got.astype(np.float64) - ref)
    scale = np.abs(ref).max()
    assert np.quantile(err, 0.999) <= q999 * scale and err.max() <= worst * scale, (np.quantile(err, 0.999) / scale, err.max() / scale)


def test_engine_small_encoder_against_oracle_and_eager_path(backend, oracle):
    enc, orc = _build(oracle, n_mels=16, state=128, heads=2, layers=3, n_ctx=56, std=0.05)
    mel = _rb(synth.normal("we-mel", (3, 16, 112)))
    tm = Tensor(mel, dtype="bfloat16")
    eng = WhisperEncoderEngine(enc)
    n0 = backend.launch_count(reset=True)
    y = eng.forward(tm)
    launches = backend.launch_count() - 0
    assert y.shape == (3, 56, 128) and y.dtype == "bfloat16"
    got = y.dataAsync()
    ref = orc.forward(mel)
    # final LayerNorm output is O(1); bf16 storage of the residual stream bounds the error
    _check(got, ref, 2e-2, 4e-2)
    eager = enc.forward(tm).dataAsync()
    # the eager path rounds after every operator: the fused path must be at least as close to the oracle
    assert np.abs(got - ref).mean() <= np.abs(eager - ref).mean() * 1.05
    _check(got, eager.astype(np.float64), 3e-2, 6e-2)
    assert launches > 0 and n0 >= 0
    # a shorter clip than the position table
    mel2 = _rb(synth.normal("we-mel2", (1, 16, 64)))
    y2 = eng.forward(Tensor(mel2, dtype="bfloat16")).dataAsync()
    _check(y2, orc.forward(mel2), 2e-2, 4e-2)


def test_engine_whisper_small_shapes_two_layers(backend, oracle):
    """80 mel bins x 3000 frames -> 1500 x 768, 12 heads of 64 (non-causal attention with a ragged
    last key tile, strided q/k/v views of the packed projection)."""
    enc, orc = _build(oracle, n_mels=80, state=768, heads=12, layers=2, n_ctx=1500, std=0.02)
    mel = _rb(synth.normal("mel", (2, 80, 3000)))
    eng = WhisperEncoderEngine(enc)
    got = eng.forward(Tensor(mel, dtype="bfloat16")).dataAsync()
    assert got.shape == (2, 1500, 768)
    _check(got, orc.forward(mel), 2e-2, 5e-2)


def test_engine_rejects_fp32_encoders(backend):
    cfg = WhisperConfig(nMels=8, nAudioCtx=20, nAudioState=128, nAudioHead=2, nAudioLayer=1)
    with pytest.raises(ValueError):
        WhisperEncoderEngine(WhisperAudioEncoder(cfg))
