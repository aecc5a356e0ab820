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


# =============================================================================================== Llama-4
def _rope_2d_angles(grid: int, head_dim: int, theta: float, device) -> torch.Tensor:
  """Angles [grid*grid + 1, head_dim/2] of the Llama-4 vision rotary embedding: the first half of a head's lane pairs
  rotates with the patch column (x + 1), the second half with the patch row (y + 1); the class token (last) is not rotated."""
  n = grid * grid
  idx = torch.arange(n, device=device)
  x, y = (idx % grid).float() + 1.0, (idx // grid).float() + 1.0
  fd = head_dim // 2
  freq = 1.0 / (theta ** (torch.arange(0, fd, 2, device=device)[: fd // 2].float() / fd))      # [head_dim/4]
  ang = torch.cat([x[:, None] * freq[None], y[:, None] * freq[None]], dim=-1)                   # [n, head_dim/2]
  return torch.cat([ang, torch.zeros(1, ang.shape[1], device=device)], dim=0)


def _rotate_pairs(t: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
  """t [B, S, H, Dh] with adjacent lane pairs (re, im); ang [S, Dh/2]."""
  tf = t.float()
  re, im = tf[..., 0::2], tf[..., 1::2]
  c, s = torch.cos(ang)[None, :, None, :], torch.sin(ang)[None, :, None, :]
  return torch.stack([re * c - im * s, re * s + im * c], dim=-1).flatten(-2).to(t.dtype)


class _Llama4EncoderLayer:
  def __init__(self, b: L.Builder, c, i: int):
    d, h = c.hidden_size_for_vit, c.num_attention_heads_for_vit
    self.h, self.dh = h, d // h
    lb = b.sub("Llama4VisionEncoder_0", f"layers_{i}")
    eps = 1e-5
    self.ln0 = L.Norm(lb, "input_layer_norm", d, eps, kind="layernorm")
    ab = lb.sub("self_attention_vision")
    mk = lambda n: ab.sub(n).linear("kernel", (d,), (h, self.dh), ("embed", "heads", "kv"))  # noqa: E731
    self.q, self.k, self.v = mk("query"), mk("key"), mk("value")
    self.o = ab.sub("out").linear("kernel", (h, self.dh), (d,), ("heads", "kv", "embed"))
    self.bq, self.bk, self.bv = (ab.sub(n).vector("bias", d, ("heads",), init="zeros") for n in ("query", "key", "value"))
    self.bo = ab.sub("out").vector("bias", d, ("embed",), init="zeros")
    self.ln1 = L.Norm(lb, "post_attention_layer_norm", d, eps, kind="layernorm")
    mb = lb.sub("Llama4VisionMLP_0")
    f = c.intermediate_size_for_vit
    self.w1 = mb.sub("vit_encoder_layer_mlp_fc1").linear("kernel", (d,), (f,), ("embed", "mlp"))
    self.b1 = mb.sub("vit_encoder_layer_mlp_fc1").vector("bias", f, ("mlp",), init="zeros")
    self.w2 = mb.sub("vit_encoder_layer_mlp_fc2").linear("kernel", (f,), (d,), ("mlp", "embed"))
    self.b2 = mb.sub("vit_encoder_layer_mlp_fc2").vector("bias", d, ("embed",), init="zeros")

  def __call__(self, x, ang):
    B, S, _ = x.shape
    y = self.ln0(x)
    q = _rotate_pairs(F.linear(y, self.q, bias=self.bq).view(B, S, self.h, self.dh), ang)
    k = _rotate_pairs(F.linear(y, self.k, bias=self.bk).view(B, S, self.h, self.dh), ang)
    v = F.linear(y, self.v, bias=self.bv).view(B, S, self.h, self.dh)
    a = ref.attention(q, k, v, None, 1.0 / math.sqrt(self.dh)).to(x.dtype)
    x = x + F.linear(a.reshape(B, S, -1), self.o, bias=self.bo)
    y = F.linear(self.ln1(x), self.w1, bias=self.b1)
    y = tF.gelu(y.float()).to(x.dtype)
    return x + F.linear(y, self.w2, bias=self.b2)


class Llama4Vision:
  """Llama-4 vision tower, pixel-shuffle adapter and projector (src/maxtext/models/llama4.py:44-300, 623-825).

  Tiles [M, 3, H, W] -> unfolded patches -> linear -> + class token (appended last) -> + positions -> LayerNorm ->
  encoder layers with the two-dimensional rotary embedding -> LayerNorm -> class token dropped -> pixel shuffle (each
  2 x 2 block of patches becomes one token with four times the channels) -> two GELU linears -> projection to the language
  model width. `__call__(tiles [B, N, 3, H, W]) -> [B, N, tokens, emb_dim]`."""

  def __init__(self, config, par: dict):
    c = self.c = config
    b = L.Builder(c, "vision", None, None, **par)
    vb = b.sub("vision_encoder", "Llama4VisionModel_0")
    P, C, d = c.patch_size_for_vit, c.num_channels_for_vit, c.hidden_size_for_vit
    tile = int(getattr(c, "tile_size_for_vit", 0) or c.image_size_for_vit)
    self.tile, self.grid = tile, tile // P
    # HF / reference unfold order: (channel, row, column) inside a patch
    self.patch = vb.sub("Llama4UnfoldConvolution_0", "vit_unfold_linear").linear("kernel", (C, P, P), (d,), (None, None, None, "embed"))
    self.cls = vb.vector("class_embedding", d, ("embed",), init="zeros")
    self.pos = vb.table("positional_embedding_vlm", (self.grid * self.grid + 1, d), (None, "embed"), init="fan_in_normal")
    self.ln_pre = L.Norm(vb, "layernorm_pre", d, 1e-5, kind="layernorm")
    self.ln_post = L.Norm(vb, "layernorm_post", d, 1e-5, kind="layernorm")
    self.layers = [_Llama4EncoderLayer(vb, c, i) for i in range(c.num_hidden_layers_for_vit)]
    r = float(c.pixel_shuffle_ratio_for_vit)
    self.ratio = r
    shuffled = int(d / (r * r))
    pin, pout = int(c.projector_input_dim_for_vit), int(c.projector_output_dim_for_vit)
    sb = vb.sub("Llama4VisionPixelShuffleMLP_0", "pixel_shuffle_mlp")
    self.fc1 = sb.sub("vit_pixel_shuffle_mlp_fc1").linear("kernel", (shuffled,), (pin,), ("embed", "mlp"))
    self.fc2 = sb.sub("vit_pixel_shuffle_mlp_fc2").linear("kernel", (pin,), (pout,), ("mlp", "embed"))
    self.proj = b.sub("vision_encoder", "Llama4MultiModalProjector_0", "vit_multi_modal_projector").linear(
        "kernel", (int(c.vision_output_dim_for_vit),), (c.emb_dim,), ("embed", "embed_out"))
    self.theta = float(c.rope_theta_for_vit)
    self.params = b.params

  def _pixel_shuffle(self, x):
    """[M, g*g, d] -> [M, (g r)^2, d / r^2]: fold neighbouring columns, then neighbouring rows, into the channel dim."""
    M, n, d = x.shape
    g, r = self.grid, self.ratio
    x = x.view(M, g, g, d)
    x = x.view(M, g, int(g * r), int(d / r))
    x = x.permute(0, 2, 1, 3).contiguous()
    x = x.view(M, int(g * r), int(g * r), int(d / (r * r)))
    x = x.permute(0, 2, 1, 3).contiguous()
    return x.view(M, -1, x.shape[-1])

  def __call__(self, tiles: torch.Tensor) -> torch.Tensor:
    B, N = tiles.shape[:2]
    dt = self.patch.data.dtype
    img = tiles.reshape(B * N, *tiles.shape[2:]).to(dt)
    M, C, H, W = img.shape
    P, g = self.c.patch_size_for_vit, self.grid
    assert H == W == g * P, f"tiles must be {g * P} x {g * P}"
    patches = img.view(M, C, g, P, g, P).permute(0, 2, 4, 1, 3, 5).reshape(M, g * g, C * P * P)
    x = F.linear(patches, self.patch)
    x = torch.cat([x, self.cls.leaf().to(dt)[None, None].expand(M, 1, -1)], dim=1) + self.pos.leaf().to(dt)[None]
    x = self.ln_pre(x)
    ang = _rope_2d_angles(g, self.layers[0].dh, self.theta, x.device)
    for lyr in self.layers:
      x = lyr(x, ang)
    x = self.ln_post(x)[:, :-1]
    x = self._pixel_shuffle(x)
    x = tF.gelu(F.linear(x, self.fc1).float()).to(dt)
    x = tF.gelu(F.linear(x, self.fc2).float()).to(dt)
    x = F.linear(x, self.proj)
    return x.view(B, N, x.shape[1], -1)


# =============================================================================================== Qwen3-VL / Qwen3-Omni
class _QwenMerger:
  """Patch merger (src/maxtext/models/qwen3.py:1672-1786): groups of merge^2 neighbouring patches are concatenated, LayerNorm
  (before or after the concatenation), Linear -> GELU -> Linear to the language model's width."""

  def __init__(self, b: L.Builder, c, name: str, post_shuffle_norm: bool, eps: float):
    d, m = c.hidden_size_for_vit, c.spatial_merge_size_for_vit ** 2
    self.m, self.d, self.post = m, d, post_shuffle_norm
    mb = b.sub(name)
    self.ln = L.Norm(mb, "ln_q", d * m if post_shuffle_norm else d, eps, kind="layernorm")
    self.w0 = mb.sub("mlp_0").linear("kernel", (d * m,), (d * m,), ("embed", "mlp"))
    self.b0 = mb.sub("mlp_0").vector("bias", d * m, ("mlp",), init="zeros")
    self.w2 = mb.sub("mlp_2").linear("kernel", (d * m,), (c.out_hidden_size_for_vit,), ("mlp", "embed"))
    self.b2 = mb.sub("mlp_2").vector("bias", c.out_hidden_size_for_vit, ("embed",), init="zeros")

  def __call__(self, x):
    """x [M, S, d] in merge order (the merge^2 patches of a block are consecutive) -> [M, S / merge^2, out]."""
    M, S, d = x.shape
    if self.post:
      x = self.ln(x.reshape(M, S // self.m, self.m * d))
    else:
      x = self.ln(x).reshape(M, S // self.m, self.m * d)
    y = tF.gelu(F.linear(x, self.w0, bias=self.b0).float()).to(x.dtype)
    return F.linear(y, self.w2, bias=self.b2)


class _QwenVisionBlock:
  def __init__(self, b: L.Builder, c, i: int, eps: float):
    d, h = c.hidden_size_for_vit, c.num_attention_heads_for_vit
    self.h, self.dh = h, d // h
    bb = b.sub(f"blocks_{i}")
    self.ln1, self.ln2 = L.Norm(bb, "ln1", d, eps, kind="layernorm"), L.Norm(bb, "ln2", d, eps, kind="layernorm")
    ab = bb.sub("attn", "attn")
    mk = lambda n: ab.sub(n).linear("kernel", (d,), (h, self.dh), ("embed", "heads", "kv"))  # noqa: E731
    self.q, self.k, self.v = mk("query"), mk("key"), mk("value")
    self.bq, self.bk, self.bv = (ab.sub(n).vector("bias", d, ("heads",), init="zeros") for n in ("query", "key", "value"))
    self.o = ab.sub("out").linear("kernel", (h, self.dh), (d,), ("heads", "kv", "embed"))
    self.bo = ab.sub("out").vector("bias", d, ("embed",), init="zeros")
    f = c.intermediate_size_for_vit
    self.w1 = bb.sub("mlp").linear("kernel", (d,), (f,), ("embed", "mlp"))
    self.b1 = bb.sub("mlp").vector("bias", f, ("mlp",), init="zeros")
    self.w2 = bb.sub("mlp_out").linear("kernel", (f,), (d,), ("mlp", "embed"))
    self.b2 = bb.sub("mlp_out").vector("bias", d, ("embed",), init="zeros")

  def __call__(self, x, cos, sin):
    M, S, _ = x.shape
    y = self.ln1(x)
    q = F.linear(y, self.q, bias=self.bq).view(M, S, self.h, self.dh)
    k = F.linear(y, self.k, bias=self.bk).view(M, S, self.h, self.dh)
    v = F.linear(y, self.v, bias=self.bv).view(M, S, self.h, self.dh)

    def rot(t):                                     # rotate-half with the (row, column) angle table
      tf = t.float()
      half = tf.shape[-1] // 2
      r = torch.cat([-tf[..., half:], tf[..., :half]], dim=-1)
      return (tf * cos + r * sin).to(t.dtype)
    a = ref.attention(rot(q), rot(k), v, None, 1.0 / math.sqrt(self.dh)).to(x.dtype)      # bidirectional within one image
    x = x + F.linear(a.reshape(M, S, -1), self.o, bias=self.bo)
    y = F.linear(self.ln2(x), self.w1, bias=self.b1)
    y = tF.gelu(y.float(), approximate="tanh").to(x.dtype)
    return x + F.linear(y, self.w2, bias=self.b2)


class Qwen3VLVision:
  """Vision tower of Qwen3-VL / Qwen3-Omni (src/maxtext/models/qwen3.py:1672-2256, qwen3_vl_vision.py, qwen3_5_vision.py).

  A frame pair [C, 2, H, W] is cut into patch_size x patch_size x temporal_patch_size patches (one linear map each, the
  reference's 3-D convolution); a learned position grid of sqrt(num_position_embeddings)^2 entries is bilinearly interpolated
  to the patch grid; blocks are pre-LayerNorm encoders with a 2-D rotary embedding (row angles on the first half of each
  rotary half, column angles on the second); tokens are kept in MERGE ORDER (the merge x merge patches that the merger will
  fuse are consecutive). The exit merger gives (H/P/merge) x (W/P/merge) soft tokens per image; the hidden states after the
  blocks listed in `deepstack_visual_indexes_for_vit` go through mergers of their own and are added to the decoder's hidden
  states at the image positions after its first layers ("deepstack").

  `__call__(images [B, N, 3, H, W]) -> [B, N, K, out_hidden]`; the deepstack features of the last call are in `.deepstack`
  (list of [B, N, K, out_hidden])."""

  def __init__(self, config, par: dict):
    c = self.c = config
    b = L.Builder(c, "vision", None, None, **par)
    vb = b.sub("vision_encoder")
    self.P, self.TP, self.C, self.d = c.patch_size_for_vit, c.temporal_patch_size_for_vit, c.num_channels_for_vit, c.hidden_size_for_vit
    self.merge = c.spatial_merge_size_for_vit
    eps = 1e-6
    # reference kernel layout of the 3-D patch convolution: [T, P, P, C, d]
    self.patch = vb.sub("patch_embed", "proj").linear("kernel", (self.TP, self.P, self.P, self.C), (self.d,), (None, None, None, None, "embed"))
    self.patch_bias = vb.sub("patch_embed", "proj").vector("bias", self.d, ("embed",), init="zeros")
    self.side = int(math.isqrt(int(c.num_position_embeddings_for_vit)))
    self.pos = vb.sub("pos_embed_interpolate").table("pos_embed", (self.side * self.side, self.d), (None, "embed"), init="fan_in_normal")
    self.blocks = [_QwenVisionBlock(vb, c, i, eps) for i in range(c.num_hidden_layers_for_vit)]
    self.deep_idx = [int(i) for i in (c.deepstack_visual_indexes_for_vit or [])]
    self.deep_mergers = [_QwenMerger(vb, c, f"merger_{i}", True, eps) for i in range(len(self.deep_idx))]
    self.merger = _QwenMerger(b.sub("vision_projector"), c, "merger", False, eps)
    self.params = b.params
    self.deepstack = []

  # ---- token order and tables
  def _merge_order(self, gh: int, gw: int, device):
    """Patch (row, col) of every token, blocks of merge x merge patches consecutive: [gh*gw, 2]."""
    m = self.merge
    br, bc = torch.arange(gh // m, device=device), torch.arange(gw // m, device=device)
    ir, ic = torch.arange(m, device=device), torch.arange(m, device=device)
    rows = (br[:, None, None, None] * m + ir[None, None, :, None]).expand(gh // m, gw // m, m, m).reshape(-1)
    cols = (bc[None, :, None, None] * m + ic[None, None, None, :]).expand(gh // m, gw // m, m, m).reshape(-1)
    return torch.stack([rows, cols], -1)

  def _pos_embed(self, rc, gh: int, gw: int):
    """Bilinear interpolation of the learned side x side grid at the patch centres (corner aligned), for tokens at `rc`."""
    s = self.side
    tab = self.pos.leaf().float()
    hi = torch.linspace(0, s - 1, gh, device=rc.device)[rc[:, 0]]
    wi = torch.linspace(0, s - 1, gw, device=rc.device)[rc[:, 1]]
    h0, w0 = hi.floor().long(), wi.floor().long()
    h1, w1 = (h0 + 1).clamp(max=s - 1), (w0 + 1).clamp(max=s - 1)
    dh, dw = (hi - h0)[:, None], (wi - w0)[:, None]
    return (tab[h0 * s + w0] * (1 - dh) * (1 - dw) + tab[h0 * s + w1] * (1 - dh) * dw +
            tab[h1 * s + w0] * dh * (1 - dw) + tab[h1 * s + w1] * dh * dw)

  def _rope(self, rc):
    """cos / sin [S, 1, head_dim]: angles = [row * f | col * f] repeated for the two rotate-half halves."""
    dh = self.d // self.c.num_attention_heads_for_vit
    inv = 1.0 / (float(self.c.rope_theta_for_vit) ** (torch.arange(0, dh // 2, 2, device=rc.device, dtype=torch.float32) / (dh // 2)))
    ang = torch.cat([rc[:, :1].float() * inv, rc[:, 1:].float() * inv], -1)           # [S, dh/2]
    ang = torch.cat([ang, ang], -1)[:, None]
    return ang.cos(), ang.sin()

  def patches(self, images: torch.Tensor) -> torch.Tensor:
    """[M, C, H, W] (one frame, repeated over the temporal patch) or [M, TP, C, H, W] (the frames of a video's temporal patch)
    -> [M, S, TP*P*P*C] in merge order, features ordered (t, py, px, c) like the reference kernel."""
    P = self.P
    if images.dim() == 5:
      # video: [M, TP, C, H, W], the frames of one temporal patch are distinct
      M, T, C, H, W = images.shape
      assert T == self.TP, f"a temporal patch holds {self.TP} frames, got {T}"
      gh, gw = H // P, W // P
      assert H % (P * self.merge) == 0 and W % (P * self.merge) == 0, "frame sides must be multiples of patch_size * spatial_merge_size"
      rc = self._merge_order(gh, gw, images.device)
      x = images.view(M, T, C, gh, P, gw, P).permute(0, 3, 5, 1, 4, 6, 2)               # M, gy, gx, t, py, px, C
      x = x[:, rc[:, 0], rc[:, 1]]
      return x.reshape(M, x.shape[1], T * P * P * C), rc, gh, gw
    M, C, H, W = images.shape
    gh, gw = H // P, W // P
    assert H % (P * self.merge) == 0 and W % (P * self.merge) == 0, "image sides must be multiples of patch_size * spatial_merge_size"
    rc = self._merge_order(gh, gw, images.device)
    x = images.view(M, C, gh, P, gw, P).permute(0, 2, 4, 3, 5, 1)                     # M, gy, gx, py, px, C
    x = x[:, rc[:, 0], rc[:, 1]]                                                      # M, S, py, px, C
    x = x.unsqueeze(2).expand(M, x.shape[1], self.TP, P, P, C)
    return x.reshape(M, x.shape[1], self.TP * P * P * C), rc, gh, gw

  def __call__(self, images: torch.Tensor) -> torch.Tensor:
    B, N = images.shape[:2]
    dt = self.patch.data.dtype
    x, rc, gh, gw = self.patches(images.reshape(B * N, *images.shape[2:]).to(dt))
    x = F.linear(x, self.patch, bias=self.patch_bias)
    x = x + self._pos_embed(rc, gh, gw).to(dt)
    cos, sin = self._rope(rc)
    deep = []
    for i, blk in enumerate(self.blocks):
      x = blk(x, cos, sin)
      if i in self.deep_idx:
        deep.append(self.deep_mergers[self.deep_idx.index(i)](x))
    out = self.merger(x)
    self.deepstack = [t.view(B, N, t.shape[1], -1) for t in deep]
    return out.view(B, N, out.shape[1], -1)


# =============================================================================================== Gemma-4
class _Gemma4EncoderBlock:
  """Sandwich-normed encoder block of the Gemma-4 tower (src/maxtext/models/gemma4_vision.py:422-533): RMS norms before and after
  both branches, q / k norms with scale and a scale-free v norm, no 1/sqrt(d) factor, a 2-D rotary embedding whose two halves of
  the head rotate by the patch's x and y coordinate, and a gated GELU MLP. The input / output clipping of the published
  checkpoints' linears is not applied."""

  def __init__(self, b: L.Builder, c, i: int):
    d, h = c.hidden_size_for_vit, c.num_attention_heads_for_vit
    self.h, self.dh, self.eps = h, d // h, c.normalization_layer_epsilon
    eb = b.sub(f"layers_{i}")
    mk = lambda n: L.Norm(eb, n, d, self.eps)  # noqa: E731
    self.n_in, self.n_post_attn, self.n_pre_ffw, self.n_post_ffw = mk("pre_attention_norm"), mk("post_attention_norm"), mk("pre_ffw_norm"), mk("post_ffw_norm")
    ab = eb.sub("attention")
    lin = lambda n: ab.sub(n).linear("kernel", (d,), (h, self.dh), ("embed", "heads", "kv"))  # noqa: E731
    self.q, self.k, self.v = lin("query"), lin("key"), lin("value")
    self.o = ab.sub("out").linear("kernel", (h, self.dh), (d,), ("heads", "kv", "embed"))
    self.qn = L.Norm(ab, "query_norm", self.dh, self.eps, axes=("norm",))
    self.kn = L.Norm(ab, "key_norm", self.dh, self.eps, axes=("norm",))
    f = c.intermediate_size_for_vit
    mb = eb.sub("mlp")
    self.w0 = mb.sub("wi_0").linear("kernel", (d,), (f,), ("embed", "mlp"))
    self.w1 = mb.sub("wi_1").linear("kernel", (d,), (f,), ("embed", "mlp"))
    self.wo = mb.sub("wo").linear("kernel", (f,), (d,), ("mlp", "embed"))

  def __call__(self, x, cos, sin):
    M, S, _ = x.shape
    y = self.n_in(x)
    q = self.qn(F.linear(y, self.q).view(M, S, self.h, self.dh))
    k = self.kn(F.linear(y, self.k).view(M, S, self.h, self.dh))
    v = F.linear(y, self.v).view(M, S, self.h, self.dh)
    vf = v.float()
    v = (vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + self.eps)).to(v.dtype)

    def rot(t):                                     # each half of the head is rotated (rotate-half inside the half) by its own axis
      tf = t.float()
      a, b2 = tf[..., :self.dh // 2], tf[..., self.dh // 2:]

      def rh(z):
        q4 = z.shape[-1] // 2
        return torch.cat([-z[..., q4:], z[..., :q4]], -1)
      out = torch.cat([a, b2], -1) * cos + torch.cat([rh(a), rh(b2)], -1) * sin
      return out.to(t.dtype)
    a = ref.attention(rot(q), rot(k), v, None, 1.0).to(x.dtype)
    x = x + self.n_post_attn(F.linear(a.reshape(M, S, -1), self.o))
    y = self.n_pre_ffw(x)
    g = tF.gelu(F.linear(y, self.w0).float(), approximate="tanh").to(x.dtype) * F.linear(y, self.w1)
    return x + self.n_post_ffw(F.linear(g, self.wo))


class Gemma4Vision:
  """Vision tower of Gemma-4 (src/maxtext/models/gemma4_vision.py:88-650): a bias-free linear map of every patch_size^2 x 3
  patch, learned x- and y-position tables that are ADDED (one row per coordinate), `num_hidden_layers_for_vit` encoder blocks,
  k x k average pooling of the patch grid down to `vision_output_length` soft tokens, a sqrt(width) scale, a scale-free RMS
  norm and the projection to the language model's width.

  `__call__(images [B, N, 3, H, W]) -> [B, N, K, emb_dim]`, images already normalised to [-1, 1]."""

  def __init__(self, config, par: dict):
    c = self.c = config
    b = L.Builder(c, "vision", None, None, **par)
    vb = b.sub("vision_encoder")
    self.P, self.d = int(c.patch_size_for_vit), int(c.hidden_size_for_vit)
    self.patch = vb.sub("entry", "input_projection").linear("kernel", (self.P, self.P, int(c.num_channels_for_vit)), (self.d,), (None, None, None, "embed"))
    self.pos_size = int(c.num_position_embeddings_for_vit)
    self.pos = vb.sub("entry").table("pos_emb", (2, self.pos_size, self.d), (None, None, "embed"), init="fan_in_normal")
    self.blocks = [_Gemma4EncoderBlock(vb, c, i) for i in range(c.num_hidden_layers_for_vit)]
    pb = b.sub("vision_projector")
    self.proj = pb.sub("projection").linear("kernel", (self.d,), (c.emb_dim,), ("embed", "embed_out"))
    self.params = b.params

  def _grid(self, H: int, W: int, device):
    gh, gw = H // self.P, W // self.P
    ys, xs = torch.meshgrid(torch.arange(gh, device=device), torch.arange(gw, device=device), indexing="ij")
    return gh, gw, torch.stack([xs.reshape(-1), ys.reshape(-1)], -1)          # (x, y) per patch, row-major

  def patches(self, images: torch.Tensor) -> torch.Tensor:
    """[M, C, H, W] -> [M, gh*gw, P*P*C], features ordered (row, column, channel) like the reference kernel."""
    M, C, H, W = images.shape
    P = self.P
    gh, gw = H // P, W // P
    return images.view(M, C, gh, P, gw, P).permute(0, 2, 4, 3, 5, 1).reshape(M, gh * gw, P * P * C)

  def rope(self, xy):
    """cos / sin [S, 1, head_dim]: the first half of the head carries the x angles, the second the y angles."""
    dh = self.d // int(self.c.num_attention_heads_for_vit)
    sp = dh // 2
    inv = 1.0 / (float(self.c.rope_theta_for_vit) ** (torch.arange(0, sp, 2, device=xy.device, dtype=torch.float32) / sp))
    parts = []
    for i in range(2):
      f = xy[:, i:i + 1].float() * inv
      parts.append(torch.cat([f, f], -1))
    ang = torch.cat(parts, -1)[:, None]
    return ang.cos(), ang.sin()

  def encode(self, patches: torch.Tensor, xy: torch.Tensor, out_len: int) -> torch.Tensor:
    """patches [M, S, P*P*C] with coordinates xy [S, 2] -> pooled soft tokens [M, out_len, d] (before the projector)."""
    dt = self.patch.data.dtype
    x = F.linear(patches.to(dt), self.patch)
    tab = self.pos.leaf().to(dt)
    x = x + tab[0][xy[:, 0]] + tab[1][xy[:, 1]]
    cos, sin = self.rope(xy)
    for blk in self.blocks:
      x = blk(x, cos, sin)
    S = x.shape[1]
    if S != out_len:
      k = int(math.isqrt(S // out_len))
      assert k * k * out_len == S, f"cannot pool {S} patches to {out_len} tokens"
      max_x = int(xy[:, 0].max()) + 1
      cell = (xy[:, 0] // k) + (max_x // k) * (xy[:, 1] // k)
      w = tF.one_hot(cell, out_len).float() / (k * k)                                   # [S, out_len]
      x = torch.einsum("sl,msd->mld", w, x.float()).to(dt)
    return x * math.sqrt(self.d)

  def project(self, soft: torch.Tensor) -> torch.Tensor:
    sf = soft.float()
    normed = (sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + self.c.normalization_layer_epsilon)).to(soft.dtype)
    return F.linear(normed, self.proj)

  def __call__(self, images: torch.Tensor) -> torch.Tensor:
    B, N = images.shape[:2]
    H, W = images.shape[-2:]
    gh, gw, xy = self._grid(H, W, images.device)
    out_len = int(self.c.vision_output_length) if int(self.c.vision_output_length) > 0 else gh * gw
    soft = self.encode(self.patches(images.reshape(B * N, *images.shape[2:])), xy, out_len)
    out = self.project(soft)
    return out.view(B, N, out.shape[1], -1)
