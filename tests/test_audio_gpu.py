"""GPU parity of the Whisper log-mel front end (framing + window, DFT as an fp32 GEMM, power, mel
projection, log10 / clamp / scale) against the oracle's restatement of the reference pipeline
(composite.ts:527-681 stft, spectrogram.ts:63-68, MelScale.ts:95-108, whisper/audio.ts:322-414)."""
import ctypes

import numpy as np
import pytest

from kandle_b200 import audio, core, lib, synth
from kandle_b200.core import Tensor

pytestmark = pytest.mark.gpu


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


def _speechlike(seconds: float, seed: str) -> np.ndarray:
    """Seeded synthetic audio with a wide dynamic range: a few decaying harmonics plus noise bursts."""
    n = int(16000 * seconds)
    t = np.arange(n, dtype=np.float64) / 16000.0
    noise = synth.normal(f"audio-{seed}", (n,), 1.0).astype(np.float64)
    x = 0.3 * np.sin(2 * np.pi * 220 * t) * np.exp(-t) + 0.1 * np.sin(2 * np.pi * 1870 * t + 1.0)
    x += 0.02 * noise * (np.sin(2 * np.pi * 0.7 * t) > 0.3)
    return x.astype(np.float32)


def test_frames_power_and_mel_match_the_oracle(backend, oracle):
    x = _speechlike(2.0, "a")
    w = audio.hann_window_host(400)
    ms = audio.MelSpectrogram(sample_rate=16000, n_fft=400, hop_length=160, n_mels=80, f_max=8000, norm="slaney", mel_scale="slaney")
    xt = Tensor(x[None])
    T = ms.frames_count(x.size)
    frames = core.empty((1, T, 400), "float32")
    lib.call("kd_stft_frames", _r(xt), _r(ms.window), 400, 160, 1, _r(frames))
    xp = np.concatenate([np.zeros(200, np.float32), x, np.zeros(200, np.float32)])
    ref_frames = xp[np.arange(T)[:, None] * 160 + np.arange(400)[None, :]] * w[None]
    assert np.array_equal(frames.dataAsync()[0], ref_frames.astype(np.float32))      # exact: one fp32 multiply
    ref_power = oracle.stft_power(x, w, 400, 160)
    spec = core.matmul(frames.view(T, 400), ms.basis)
    power = core.empty((T, 201), "float32")
    lib.call("kd_power_spectrum", _r(spec), _r(power))
    got = power.dataAsync()
    # a 400-term fp32 DFT against the exactly rounded one: relative to the frame's strongest bin
    assert np.abs(got - ref_power).max() <= 2e-5 * ref_power.max()
    mel = ms.forward(xt).dataAsync()[0]
    fb = audio.melscale_fbanks_host(201, 0, 8000, 80, 16000, "slaney", "slaney")
    ref_mel = (ref_power.astype(np.float64) @ fb.astype(np.float64)).T
    assert mel.shape == (80, T)
    assert np.abs(mel - ref_mel).max() <= 2e-5 * ref_mel.max()


@pytest.mark.parametrize("seconds", [30.0, 7.3, 0.01])
def test_whisper_features_match_the_oracle(backend, oracle, seconds):
    x = _speechlike(seconds, f"w{seconds}")
    fe = audio.WhisperFeatureExtractor(80)
    got = fe.extract(x, 16000).dataAsync()
    ref = oracle.whisper_log_mel(x, audio.hann_window_host(400), audio.melscale_fbanks_host(201, 0, 8000, 80, 16000, "slaney", "slaney"))
    assert got.shape == ref.shape == (1, 80, 3000)
    # outputs are (log10 + 4) / 4: 1e-4 here is 4e-4 in log10, i.e. 0.1 % in power
    err = np.abs(got - ref)
    assert err.max() <= 1e-3 and np.sqrt((err ** 2).mean()) <= 2e-5, f"max {err.max():.2e} rms {np.sqrt((err ** 2).mean()):.2e}"
    # silence (zero padding to 30 s) sits exactly on the clamp floor
    if seconds < 29:
        floor = ref.min()
        assert np.all(got[0, :, -100:] == floor)


def test_features_feed_the_encoder_shapes(backend):
    """[1, 80, 3000] is what WhisperAudioEncoder.forward takes (conv1 stride 1, conv2 stride 2 -> 1500 positions)."""
    fe = audio.WhisperFeatureExtractor(80)
    out = fe.extract(_speechlike(1.0, "enc"), 16000)
    assert out.shape == (1, 80, 3000) and out.dtype == "float32"
    with pytest.raises(NotImplementedError):
        fe.extract(np.zeros(100, np.float32), 44100)


def test_argument_checks(backend):
    x = Tensor(np.zeros((1, 1000), np.float32))
    w = Tensor(np.ones(400, np.float32))
    bad = core.empty((1, 5, 400), "float32")
    with pytest.raises(lib.KandleCudaError):
        lib.call("kd_stft_frames", _r(x), _r(w), 400, 160, 1, _r(bad))       # 7 frames expected
    with pytest.raises(lib.KandleCudaError):
        lib.call("kd_power_spectrum", _r(bad), _r(core.empty((1, 5, 201), "float32")))   # 400 != 2*201
