"""Vision tower and projector of Gemma-3 (src/maxtext/models/gemma3.py:368-732, src/maxtext/layers/encoders.py:27-211).

An image [3, H, W] is cut into patch_size x patch_size patches, each patch is one linear map to the tower width (the
reference's strided convolution), a learned position table is added, and `num_hidden_layers_for_vit` pre-LayerNorm
encoder blocks (bidirectional multi-head attention with biases, GELU MLP) run over the (H / patch)^2 tokens. The exit
average-pools the token grid to 256 "soft tokens" per image; the embedder RMS-normalises them and projects to the
language model's width. The decoder then sees those vectors at the positions of the image placeholder tokens.

The tower is one parameter unit ("vision"); with `freeze_vision_encoder_params` (the default) it runs without
gradient and its parameters are frozen.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as tF

from ..layers import blocks as L
from ..ops import functional as F
from ..ops import reference as ref


class _EncoderBlock:
  def __init__(self, b: L.Builder, c, i: int):
    d, h = c.hidden_size_for_vit, c.num_attention_heads_for_vit
    self.h, self.dh = h, d // h
    eb = b.sub("Transformer", f"encoderblock_{i}")
    eps = c.normalization_layer_epsilon
    self.ln0 = L.Norm(eb, "LayerNorm_0", d, eps, kind="layernorm")
    ab = eb.sub("MultiHeadDotProductAttention_0")
    mk = lambda n, tp: ab.sub(n).linear("kernel", (d,), (h, self.dh), ("embed", "heads", "kv"))  # noqa: E731
    self.q, self.k, self.v = mk("query", None), mk("key", None), mk("value", None)
    self.o = ab.sub("out").linear("kernel", (h, self.dh), (d,), ("heads", "kv", "embed"))
    self.bq, self.bk, self.bv = (ab.sub(n).vector("bias", d, ("heads",), init="zeros") for n in ("query", "key", "value"))
    self.bo = ab.sub("out").vector("bias", d, ("embed",), init="zeros")
    self.ln1 = L.Norm(eb, "LayerNorm_1", d, eps, kind="layernorm")
    mb = eb.sub("MlpBlockViT_0")
    f = c.intermediate_size_for_vit
    self.w1 = mb.sub("Dense_0").linear("kernel", (d,), (f,), ("embed", "mlp"))
    self.b1 = mb.sub("Dense_0").vector("bias", f, ("mlp",), init="zeros")
    self.w2 = mb.sub("Dense_1").linear("kernel", (f,), (d,), ("mlp", "embed"))
    self.b2 = mb.sub("Dense_1").vector("bias", d, ("embed",), init="zeros")

  def __call__(self, x):
    B, S, _ = x.shape
    y = self.ln0(x)
    q = F.linear(y, self.q, bias=self.bq).view(B, S, self.h, self.dh)
    k = F.linear(y, self.k, bias=self.bk).view(B, S, self.h, self.dh)
    v = F.linear(y, self.v, bias=self.bv).view(B, S, self.h, self.dh)
    a = ref.attention(q, k, v, None, 1.0 / math.sqrt(self.dh)).to(x.dtype)
    x = x + F.linear(a.reshape(B, S, -1), self.o, bias=self.bo)
    y = self.ln1(x)
    y = F.linear(y, self.w1, bias=self.b1)
    y = tF.gelu(y.float(), approximate="tanh").to(x.dtype)
    return x + F.linear(y, self.w2, bias=self.b2)


class Gemma3Vision:
  """Encoder + exit + embedder. `__call__(images [B, N, 3, H, W]) -> [B, N, 256, emb_dim]`."""

  TOKENS_PER_IMAGE = 256

  def __init__(self, config, par: dict):
    c = config
    self.c = c
    b = L.Builder(c, "vision", None, None, **par)
    vb = b.sub("vision_encoder", "Gemma3VisionEncoderLayer_0")
    P, C, d = c.patch_size_for_vit, c.num_channels_for_vit, c.hidden_size_for_vit
    assert c.conv_stride_for_vit == P, "patches must not overlap"
    self.grid = c.image_size_for_vit // P
    # the patch convolution as a linear map over flattened patches, reference kernel layout [P, P, C, d]
    self.patch = vb.sub("embedding").linear("kernel", (P, P, C), (d,), (None, None, None, "embed"))
    self.patch_bias = vb.sub("embedding").vector("bias", d, ("embed",), init="zeros")
    self.pos = vb.table("pos_embedding", (1, self.grid * self.grid, d), (None, None, "embed"), init="fan_in_normal")
    self.blocks = [_EncoderBlock(vb, c, i) for i in range(c.num_hidden_layers_for_vit)]
    self.final = L.Norm(vb.sub("Transformer"), "encoder_norm", d, c.normalization_layer_epsilon, kind="layernorm")
    eb = b.sub("vision_encoder", "VisionEmbedder_0")
    self.soft_norm = L.Norm(eb, "mm_soft_embedding_norm", d, c.normalization_layer_epsilon)
    self.proj = eb.sub("mm_input_projection").linear("w", (d,), (c.emb_dim,), ("embed", "embed_out"))
    self.params = b.params

  def patches(self, images: torch.Tensor) -> torch.Tensor:
    """[M, C, H, W] -> [M, grid*grid, P*P*C] with the (row, column, channel) order of the reference kernel."""
    M, C, H, W = images.shape
    P, g = self.c.patch_size_for_vit, self.grid
    assert H == W == g * P, f"images must be {g * P} x {g * P}"
    x = images.view(M, C, g, P, g, P).permute(0, 2, 4, 3, 5, 1)          # M, gy, gx, py, px, C
    return x.reshape(M, g * g, P * P * C)

  def __call__(self, images: torch.Tensor) -> torch.Tensor:
    B, N = images.shape[:2]
    dt = self.patch.data.dtype
    x = self.patches(images.reshape(B * N, *images.shape[2:]).to(dt))
    x = F.linear(x, self.patch, bias=self.patch_bias) + self.pos.leaf().to(dt)
    for blk in self.blocks:
      x = blk(x)
    x = self.final(x)
    g = self.grid
    out_w = int(math.isqrt(self.TOKENS_PER_IMAGE))
    if g * g != self.TOKENS_PER_IMAGE:
      assert g % out_w == 0
      x = tF.avg_pool2d(x.view(B * N, g, g, -1).permute(0, 3, 1, 2).float(), g // out_w).permute(0, 2, 3, 1).reshape(B * N, out_w * out_w, -1).to(dt)
    x = F.linear(self.soft_norm(x), self.proj)
    return x.view(B, N, x.shape[1], -1)
