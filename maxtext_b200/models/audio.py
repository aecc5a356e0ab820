"""Audio tower of Qwen3-Omni (src/maxtext/models/qwen3.py:2281-2590).

A log-mel spectrogram [mel bins, frames] is cut into chunks of 2 * n_window frames; every chunk goes through three stride-2
3 x 3 convolutions (GELU) over (mel, time), is flattened per time step and projected to the tower width, and gets sinusoidal
positions that restart in every chunk. The valid time steps of all chunks are concatenated and run through pre-LayerNorm
encoder layers whose attention is bidirectional inside windows of n_window_infer / (2 * n_window) chunks; a LayerNorm and a
two-layer GELU head give `output_dim_for_audio` features per time step (one soft token each).

`__call__(features [mel, frames]) -> [tokens, output_dim]` for one clip (the clips of a batch are encoded one by one).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as tF

from ..layers import blocks as L
from ..ops import functional as F
from ..ops import reference as ref


def _after_convs(n: int) -> int:
  for _ in range(3):
    n = (n - 1) // 2 + 1 if n > 0 else 0
  return n


def conv_output_length(n: int, chunk: int = 100) -> int:
  """Soft tokens of a clip of n mel frames: every chunk of `chunk` frames (and the shorter tail) is halved three times,
  rounding up (13 tokens per 100 frames)."""
  return (n // chunk) * _after_convs(chunk) + _after_convs(n % chunk)


class _AudioLayer:
  def __init__(self, b: L.Builder, c, i: int):
    d, h, f = c.d_model_for_audio, c.encoder_attention_heads_for_audio, c.encoder_ffn_dim_for_audio
    self.h, self.dh = h, d // h
    eb = b.sub(f"layers_{i}")
    self.ln1 = L.Norm(eb, "self_attn_layer_norm", d, 1e-5, kind="layernorm")
    self.ln2 = L.Norm(eb, "final_layer_norm", d, 1e-5, kind="layernorm")
    ab = eb.sub("self_attn")
    lin = lambda n: (ab.sub(n).linear("kernel", (d,), (d,), ("embed", "heads")), ab.sub(n).vector("bias", d, ("heads",), init="zeros"))  # noqa: E731
    (self.q, self.bq), (self.k, self.bk), (self.v, self.bv), (self.o, self.bo) = lin("query"), lin("key"), lin("value"), lin("out")
    self.w1, self.b1 = eb.sub("fc1").linear("kernel", (d,), (f,), ("embed", "mlp")), eb.sub("fc1").vector("bias", f, ("mlp",), init="zeros")
    self.w2, self.b2 = eb.sub("fc2").linear("kernel", (f,), (d,), ("mlp", "embed")), eb.sub("fc2").vector("bias", d, ("embed",), init="zeros")

  def __call__(self, x, mask):
    S = x.shape[0]
    y = self.ln1(x)
    q = F.linear(y, self.q, bias=self.bq).view(1, S, self.h, self.dh)
    k = F.linear(y, self.k, bias=self.bk).view(1, S, self.h, self.dh)
    v = F.linear(y, self.v, bias=self.bv).view(1, S, self.h, self.dh)
    a = ref.attention(q, k, v, mask, self.dh ** -0.5).to(x.dtype).reshape(S, -1)
    x = x + F.linear(a, self.o, bias=self.bo)
    y = tF.gelu(F.linear(self.ln2(x), self.w1, bias=self.b1).float()).to(x.dtype)
    return x + F.linear(y, self.w2, bias=self.b2)


class Qwen3OmniAudio:
  def __init__(self, config, par: dict):
    c = self.c = config
    b = L.Builder(c, "audio", None, None, **par)
    ab = b.sub("audio_encoder")
    d, ch, mel = c.d_model_for_audio, c.downsample_hidden_size_for_audio, c.num_mel_bins_for_audio
    self.d, self.nw = d, int(c.n_window_for_audio)
    conv = lambda n, cin: (ab.sub(n).table("kernel", (ch, cin, 3, 3), (None, None, None, None), init="fan_in_normal"),  # noqa: E731
                           ab.sub(n).vector("bias", ch, (None,), init="zeros"))
    self.convs = [conv("conv2d1", 1), conv("conv2d2", ch), conv("conv2d3", ch)]
    mel_out = (((mel + 1) // 2 + 1) // 2 + 1) // 2
    self.conv_out = ab.sub("conv_out").linear("kernel", (ch * mel_out,), (d,), (None, "embed"))
    self.layers = [_AudioLayer(ab, c, i) for i in range(c.encoder_layers_for_audio)]
    self.ln_post = L.Norm(ab, "ln_post", d, 1e-5, kind="layernorm")
    pb = b.sub("audio_projector")
    self.p1, self.pb1 = pb.sub("proj1").linear("kernel", (d,), (d,), ("embed", "mlp")), pb.sub("proj1").vector("bias", d, ("mlp",), init="zeros")
    self.p2 = pb.sub("proj2").linear("kernel", (d,), (c.output_dim_for_audio,), ("mlp", "embed"))
    self.pb2 = pb.sub("proj2").vector("bias", c.output_dim_for_audio, ("embed",), init="zeros")
    self.params = b.params

  def positions(self, n: int, device) -> torch.Tensor:
    half = self.d // 2
    inc = math.log(float(self.c.max_timescale_for_audio)) / (half - 1)
    inv = torch.exp(-inc * torch.arange(half, device=device, dtype=torch.float32))
    t = torch.arange(n, device=device, dtype=torch.float32)[:, None] * inv[None]
    return torch.cat([torch.sin(t), torch.cos(t)], 1)

  def __call__(self, features: torch.Tensor) -> torch.Tensor:
    dt = self.conv_out.data.dtype
    mel, n = features.shape
    win = 2 * self.nw
    chunks = list(features.t().split(win, dim=0))                                  # [frames_i, mel]
    lens = [ch.shape[0] for ch in chunks]
    padded = torch.nn.utils.rnn.pad_sequence(chunks, batch_first=True).transpose(1, 2).unsqueeze(1).to(dt)   # [chunks, 1, mel, win]
    x = padded
    for w, bias in self.convs:
      x = tF.gelu(tF.conv2d(x, w.leaf().to(dt), bias.leaf().to(dt), stride=2, padding=1))
    nb, ch_, f_, t_ = x.shape
    x = F.linear(x.permute(0, 3, 1, 2).reshape(nb, t_, ch_ * f_), self.conv_out)
    x = x + self.positions(t_, x.device).to(dt)
    after = [_after_convs(v) for v in lens]
    x = torch.cat([x[i, :after[i]] for i in range(nb)], 0)                          # valid steps of every chunk, in order
    S = x.shape[0]
    # attention windows: n_window_infer / (2 n_window) chunks' worth of time steps
    w_len = t_ * max(1, int(self.c.n_window_infer_for_audio) // win)
    block = torch.arange(S, device=x.device) // w_len
    mask = (block[:, None] == block[None, :])[None, None]
    for layer in self.layers:
      x = layer(x, mask)
    x = self.ln_post(x)
    x = tF.gelu(F.linear(x, self.p1, bias=self.pb1).float()).to(dt)
    return F.linear(x, self.p2, bias=self.pb2)
