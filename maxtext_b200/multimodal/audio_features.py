"""Waveform -> log-mel spectrogram for the Qwen3-Omni audio tower (src/maxtext/multimodal/processor_qwen3_omni.py:589-634,
the Whisper front end): 16 kHz mono, 25 ms Hann windows (400 samples) every 10 ms (160 samples), power spectrum, 128 triangular
mel filters on Slaney's scale (linear below 1 kHz, logarithmic above) with area normalisation, log10, the last frame dropped,
values floored at (max - 8) and mapped by (x + 4) / 4.

`log_mel(waveform)` returns [128, frames]; `prepare_audio(waveform, config)` pads the clip to whole 1-second units, extracts the
features and returns them with the number of soft tokens they will occupy (13 per 100 frames)."""
from __future__ import annotations

import math

import numpy as np
import torch

SAMPLE_RATE, N_FFT, HOP, N_MELS = 16000, 400, 160, 128


def _hz_to_mel(f):
  f = np.asarray(f, dtype=np.float64)
  lin = f / (200.0 / 3.0)
  log = 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (math.log(6.4) / 27.0)
  return np.where(f >= 1000.0, log, lin)


def _mel_to_hz(m):
  m = np.asarray(m, dtype=np.float64)
  lin = m * (200.0 / 3.0)
  log = 1000.0 * np.exp((m - 15.0) * (math.log(6.4) / 27.0))
  return np.where(m >= 15.0, log, lin)


def mel_filters(n_mels: int = N_MELS, n_fft: int = N_FFT, sr: int = SAMPLE_RATE, f_min: float = 0.0, f_max: float = 8000.0) -> torch.Tensor:
  """[n_fft / 2 + 1, n_mels] triangular filters, each scaled by 2 / (its band width in Hz)."""
  freqs = np.linspace(0.0, sr / 2.0, n_fft // 2 + 1)
  edges = _mel_to_hz(np.linspace(_hz_to_mel(f_min), _hz_to_mel(f_max), n_mels + 2))
  up = (freqs[:, None] - edges[None, :-2]) / (edges[1:-1] - edges[:-2])[None]
  down = (edges[None, 2:] - freqs[:, None]) / (edges[2:] - edges[1:-1])[None]
  tri = np.maximum(0.0, np.minimum(up, down))
  tri *= (2.0 / (edges[2:] - edges[:-2]))[None]
  return torch.from_numpy(tri).float()


def log_mel(waveform, n_mels: int = N_MELS) -> torch.Tensor:
  w = torch.as_tensor(np.asarray(waveform), dtype=torch.float32).reshape(-1)
  window = torch.hann_window(N_FFT, periodic=True)
  spec = torch.stft(w, N_FFT, HOP, window=window, center=True, pad_mode="reflect", return_complex=True)
  power = spec.abs() ** 2                                                  # [bins, frames + 1]
  mel = mel_filters(n_mels).t() @ power[:, :-1]
  x = torch.log10(mel.clamp_min(1e-10))
  x = torch.maximum(x, x.max() - 8.0)
  return (x + 4.0) / 4.0


def prepare_audio(waveform, config=None):
  """(features [mel, frames], number of soft tokens). The clip is zero-padded to a whole number of seconds, so the frame count
  is a multiple of 100 and every chunk of the tower is full."""
  from ..models.audio import conv_output_length
  w = np.asarray(waveform, dtype=np.float32).reshape(-1)
  unit = SAMPLE_RATE
  pad = (-len(w)) % unit
  if pad or len(w) == 0:
    w = np.pad(w, (0, pad if len(w) else unit))
  n_mels = int(getattr(config, "num_mel_bins_for_audio", N_MELS) or N_MELS) if config is not None else N_MELS
  feats = log_mel(w, n_mels)
  chunk = 2 * int(getattr(config, "n_window_for_audio", 50) or 50) if config is not None else 100
  return feats, conv_output_length(feats.shape[1], chunk)
