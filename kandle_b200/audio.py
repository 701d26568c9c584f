"""Mirror of the reference's audio front end for the Whisper path: `hannWindow`, `melscaleFbanks`,
`MelSpectrogram` (packages/core/src/audio/transforms/MelSpectrogram.ts, Spectrogram.ts,
MelScale.ts, audio/functional/filterbank.ts:88-150) and `WhisperFeatureExtractor`
(playground-node/src/whisper/audio.ts:253-414), computed on the device: framing + window in one
kernel, the 400-point DFT as an fp32 GEMM with a precomputed basis, power, mel projection, and the
log10 / clamp / scale step the reference runs in a host loop."""
from __future__ import annotations

import ctypes
import math

import numpy as np

from . import core, lib
from .core import Tensor

WHISPER_AUDIO_CONFIG = {"SAMPLE_RATE": 16000, "N_FFT": 400, "HOP_LENGTH": 160, "CHUNK_LENGTH": 30, "N_SAMPLES": 480000}


def _r(t):
    return ctypes.byref(t._handle.c()) if t is not None else None


def hann_window_host(window_length: int, periodic: bool | None = None) -> np.ndarray:
    """w[n] = 0.5 - 0.5 cos(2 pi n / M).  M follows the reference's dispatcher
    (packages/core/src/dispatch/handlers/windowfunc.ts:22-37): window_length when periodic is true,
    window_length - 1 when it is false OR NOT GIVEN -- the transforms call hannWindow(win_length)
    without the flag (Spectrogram.ts:77), so the Whisper path gets the symmetric window."""
    m = window_length if periodic else window_length - 1
    n = np.arange(window_length, dtype=np.float64)
    return (0.5 - 0.5 * np.cos(2.0 * np.pi * n / max(m, 1))).astype(np.float32)


def hannWindow(windowLength: int, periodic: bool | None = None) -> Tensor:
    return Tensor(hann_window_host(windowLength, periodic))


def _hz_to_mel_slaney(hz: float) -> float:      # filterbank.ts:33-44
    f_sp = 200.0 / 3.0
    min_log_hz = 1000.0
    min_log_mel = min_log_hz / f_sp
    logstep = math.log(6.4) / 27.0
    return min_log_mel + math.log(hz / min_log_hz) / logstep if hz >= min_log_hz else hz / f_sp


def _mel_to_hz_slaney(mel: float) -> float:     # filterbank.ts:49-60
    f_sp = 200.0 / 3.0
    min_log_hz = 1000.0
    min_log_mel = min_log_hz / f_sp
    logstep = math.log(6.4) / 27.0
    return min_log_hz * math.exp(logstep * (mel - min_log_mel)) if mel >= min_log_mel else f_sp * mel


def melscale_fbanks_host(n_freqs: int, f_min: float, f_max: float, n_mels: int, sample_rate: int, norm: str | None = None,
                         mel_scale: str = "htk") -> np.ndarray:
    """[n_freqs, n_mels] triangular filters, filterbank.ts:88-150, including its Float32Array
    storage of the band edges and bin frequencies."""
    if mel_scale == "htk":
        hz_to_mel = lambda hz: 2595.0 * math.log10(1.0 + hz / 700.0)  # noqa: E731
        mel_to_hz = lambda mel: 700.0 * (math.pow(10.0, mel / 2595.0) - 1.0)  # noqa: E731
    else:
        hz_to_mel, mel_to_hz = _hz_to_mel_slaney, _mel_to_hz_slaney
    mel_min, mel_max = hz_to_mel(f_min), hz_to_mel(f_max)
    pts = np.array([mel_to_hz(mel_min + (mel_max - mel_min) * i / (n_mels + 1)) for i in range(n_mels + 2)], dtype=np.float32)
    freqs = np.array([(sample_rate / 2) * i / (n_freqs - 1) for i in range(n_freqs)], dtype=np.float32)
    fb = np.zeros((n_freqs, n_mels), dtype=np.float32)
    f = freqs.astype(np.float64)
    for m in range(n_mels):
        left, center, right = float(pts[m]), float(pts[m + 1]), float(pts[m + 2])
        up = (f >= left) & (f <= center)
        down = (f > center) & (f <= right)
        col = np.zeros(n_freqs, dtype=np.float64)
        col[up] = (f[up] - left) / (center - left)
        col[down] = (right - f[down]) / (right - center)
        col = col.astype(np.float32)
        if norm == "slaney" and right - left > 0:
            col = (col.astype(np.float64) * (2.0 / (right - left))).astype(np.float32)
        fb[:, m] = col
    return fb


def melscaleFbanks(n_freqs, f_min, f_max, n_mels, sample_rate, norm=None, mel_scale="htk") -> Tensor:
    return Tensor(melscale_fbanks_host(n_freqs, f_min, f_max, n_mels, sample_rate, norm, mel_scale))


def dft_basis_host(n_fft: int) -> np.ndarray:
    """[n_fft, 2F]: column k < F holds cos(2 pi k n / n_fft), column F + k holds -sin(...), so that
    frames @ basis = (real parts | imaginary parts) of the one-sided DFT."""
    F = n_fft // 2 + 1
    n = np.arange(n_fft, dtype=np.float64)[:, None]
    k = np.arange(F, dtype=np.float64)[None, :]
    ang = 2.0 * np.pi * ((n * k) % n_fft) / n_fft
    return np.concatenate([np.cos(ang), -np.sin(ang)], axis=1).astype(np.float32)


class MelSpectrogram:
    """MelSpectrogram.forward of the reference: Spectrogram (power) followed by MelScale."""

    def __init__(self, sample_rate: int = 16000, n_fft: int = 400, hop_length: int | None = None, n_mels: int = 128,
                 f_min: float = 0.0, f_max: float | None = None, power: float = 2.0, norm: str | None = None,
                 mel_scale: str = "htk", center: bool = True):
        if power != 2.0:
            raise NotImplementedError("only the power spectrogram (power = 2) is on this path")
        self.n_fft, self.hop_length, self.n_mels, self.center = n_fft, hop_length or n_fft // 2, n_mels, center
        self.n_freqs = n_fft // 2 + 1
        self.window = hannWindow(n_fft)
        self.basis = Tensor(dft_basis_host(n_fft))
        self.fb = melscaleFbanks(self.n_freqs, f_min, f_max if f_max is not None else sample_rate / 2, n_mels, sample_rate,
                                 norm, mel_scale)

    def frames_count(self, length: int) -> int:
        pad = self.n_fft // 2 if self.center else 0
        return 1 + (length + 2 * pad - self.n_fft) // self.hop_length

    def mel_time_major(self, waveform: Tensor) -> Tensor:
        """[B, L] -> mel power [B, T, n_mels] (time-major: the layout the projection produces)."""
        B, L = waveform.shape
        T = self.frames_count(L)
        frames = core.empty((B, T, self.n_fft), "float32")
        lib.call("kd_stft_frames", _r(waveform), _r(self.window), self.n_fft, self.hop_length, 1 if self.center else 0, _r(frames))
        flat = frames.view(B * T, self.n_fft)
        spec = core.matmul(flat, self.basis)                      # [B*T, 2F]
        power = core.empty((B * T, self.n_freqs), "float32")
        lib.call("kd_power_spectrum", _r(spec), _r(power))
        mel = core.matmul(power, self.fb)                          # [B*T, M]
        out = mel.view(B, T, self.n_mels)
        for t in (frames, flat, spec, power):
            t.dispose()
        return out

    def forward(self, waveform: Tensor) -> Tensor:
        """[B, L] -> [B, n_mels, T], the reference's output layout (a transposed view)."""
        return self.mel_time_major(waveform).permute([0, 2, 1])


class WhisperFeatureExtractor:
    """extract(): pad or cut to 30 s, mel power spectrogram (slaney scale and norm, f_max 8000), drop the
    last frame, log10 / clamp / scale (audio.ts:322-414).  Resampling is not on this path: the input
    must already be 16 kHz."""

    def __init__(self, nMels: int = 80):
        c = WHISPER_AUDIO_CONFIG
        self.sampleRate, self.nFft, self.hopLength, self.nMels, self.nSamples = (c["SAMPLE_RATE"], c["N_FFT"], c["HOP_LENGTH"],
                                                                                nMels, c["N_SAMPLES"])
        self.melSpectrogram = MelSpectrogram(sample_rate=self.sampleRate, n_fft=self.nFft, hop_length=self.hopLength,
                                             n_mels=nMels, power=2.0, f_max=8000, norm="slaney", mel_scale="slaney")

    def extract(self, samples: np.ndarray, origSampleRate: int = 16000) -> Tensor:
        if origSampleRate != self.sampleRate:
            raise NotImplementedError("resampling is outside the accelerated path: pass 16 kHz audio")
        x = np.zeros((1, self.nSamples), dtype=np.float32)
        s = np.asarray(samples, dtype=np.float32).reshape(-1)[: self.nSamples]
        x[0, : s.size] = s
        mel = self.melSpectrogram.mel_time_major(Tensor(x))        # [1, 3001, M]
        keep = min(mel.shape[1], self.nSamples // self.hopLength)  # 3000: the last frame is dropped
        out = core.empty((1, self.nMels, keep), "float32")
        lib.call("kd_whisper_log_mel_norm", _r(mel), _r(out))
        mel.dispose()
        return out
