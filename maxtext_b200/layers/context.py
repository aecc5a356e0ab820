"""Per-call state handed to every layer: token geometry, parallel groups, remat bookkeeping, caches."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

# tensors a remat policy may keep, by policy name (src/maxtext/layers/nnx_decoders.py:1140-1268)
_PROJ = ("query_proj", "key_proj", "value_proj", "kv_proj", "qkv_proj", "out_proj")
_MLP = ("mlpwi_0", "mlpwi_1", "mlpwi", "mlpwo")
REMAT_SAVED = {
    "full": (),
    "minimal": _PROJ + _MLP,
    "minimal_with_context": _PROJ + _MLP + ("context",),
    "minimal_flash": _PROJ + _MLP + ("context",),
    "minimal_with_quantization": _PROJ + _MLP,
    "minimal_with_context_and_quantization": _PROJ + _MLP + ("context",),
    "save_dot_except_mlp": _PROJ,
    "save_dot_with_context_except_mlp": _PROJ + ("context",),
    "save_dot_except_mlpwi": _PROJ + ("mlpwo",),
    "save_qkv_proj": ("query_proj", "key_proj", "value_proj", "qkv_proj"),
    "save_out_proj": ("out_proj",),
    "qkv_proj_offloaded": (),
    "minimal_offloaded": (),
    "custom": (),
}
REMAT_OFFLOADED = {
    "qkv_proj_offloaded": ("query_proj", "key_proj", "value_proj", "qkv_proj"),
    "minimal_offloaded": _PROJ + _MLP,
}


def saved_names(config) -> tuple[tuple, tuple]:
  """(kept on device, kept on pinned host) tensor names for config.remat_policy."""
  pol = config.remat_policy
  dev = tuple(REMAT_SAVED.get(pol, ()))
  off = tuple(REMAT_OFFLOADED.get(pol, ()))
  if pol == "custom":
    dev = tuple(config.tensors_on_device)
    off = tuple(config.tensors_to_offload)
  return dev, off


@dataclass
class LayerCtx:
  config: object
  positions: torch.Tensor            # [B, S] original token positions
  segment_ids: torch.Tensor | None   # [B, S] (0 = padding)
  mode: str = "train"                # train | prefill | decode
  mesh: object = None
  tp_group: object = None
  tp_size: int = 1
  ep_group: object = None
  ep_size: int = 1
  cp_group: object = None       # ranks along `context`
  cp_size: int = 1              # total sequence split: context x context_usp_ulysses
  usp_group: object = None      # ranks along `context_usp_ulysses`
  max_logits: dict | None = None  # QK-clip: (layer, module) -> per-head maximum attention logit of this step
  expert_counts: dict | None = None  # DeepSeek bias update: MoE module -> tokens routed to each expert this step
  # remat: first forward stores named tensors, recompute forward consumes them
  save_names: tuple = ()
  offload_names: tuple = ()
  saved: dict | None = None          # name -> tensor for the current layer
  recompute: bool = False
  layer_index: int = 0
  aux_losses: list = field(default_factory=list)   # (name, tensor) produced by layers (e.g. moe_lb_loss)
  metrics: dict = field(default_factory=dict)
  cache: object = None               # inference KV cache for the current layer
  tokens: torch.Tensor | None = None
  dropout_seed: int | None = None    # training with dropout_rate > 0: base of the per-site mask seeds of this micro-batch
  sp: bool = False                   # residual stream split along the sequence over the tensor ranks (parallel.sequence_parallel)
  bidir: torch.Tensor | None = None  # [B, 1, S, S] extra allowed (query, key) pairs: tokens of one image see each other
  positions3: torch.Tensor | None = None  # [B, S, 3] (temporal, height, width) positions of a multimodal prompt (`use_mrope`)
  deepstack: tuple | None = None     # (image mask [B, S], [features [B, N*K, D], ...]): feature i is added after decoder layer i
  name_prefix: str = ""              # disambiguates blocks that share a layer (gemma2 local/global)
  batch_split: int = 1               # > 1: every decoder layer runs the batch as that many micro-batches on alternating streams
  micro_slot: int = 0                # which micro-batch of a split layer this context describes
  split_active: bool = False         # this context is one micro-batch of a split layer (its twin may run on another stream)

  def micro(self, j: int, n: int) -> "LayerCtx":
    """Context of micro-batch j of n: the per-row tensors are sliced, kept tensors go to a dictionary of their own, and
    the lists / dictionaries that a layer appends to are private so that the caller can merge them afterwards."""
    import dataclasses

    def cut(t):
      return None if t is None else t.chunk(n, 0)[j]
    sub = dataclasses.replace(self, positions=cut(self.positions), segment_ids=cut(self.segment_ids), tokens=cut(self.tokens),
                              bidir=cut(self.bidir), positions3=cut(self.positions3), batch_split=1, micro_slot=j, split_active=True, aux_losses=[],
                              max_logits={} if self.max_logits is not None else None)
    if self.deepstack is not None:
      sub.deepstack = (cut(self.deepstack[0]), [cut(f) for f in self.deepstack[1]])
    sub.saved = None if self.saved is None else self.saved.setdefault(f"mb{j}", {})
    return sub

  def dropout(self, t: torch.Tensor, site: int) -> torch.Tensor:
    """Inverted dropout whose mask depends only on (seed of the micro-batch, layer, block, site): the recompute pass of a
    rematerialised layer draws the same mask as the first pass, and tensor-parallel ranks (same seed) agree on it."""
    rate = float(getattr(self.config, "dropout_rate", 0.0) or 0.0)
    if self.dropout_seed is None or rate <= 0.0 or self.mode != "train":
      return t
    g = torch.Generator(device=t.device)
    g.manual_seed((self.dropout_seed * 1000003 + self.layer_index * 1009 + (hash(self.name_prefix) % 97) * 31 + site + 7 * self.micro_slot) % (2 ** 62))
    keep = (torch.rand(t.shape, generator=g, device=t.device) >= rate).to(t.dtype)
    return t * keep / (1.0 - rate)

  def wants(self, name: str) -> bool:
    """True in the first forward of a rematerialised layer when the policy keeps `name`."""
    return self.saved is not None and not self.recompute and (name in self.save_names or name in self.offload_names)

  def keep(self, name: str, t: torch.Tensor) -> torch.Tensor:
    """Called on a named intermediate in the first (no-grad) forward of a rematerialised layer."""
    if self.saved is not None and not self.recompute:
      if name in self.save_names:
        self.saved[self.name_prefix + name] = t
      elif name in self.offload_names:
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=t.is_cuda)
        host.copy_(t, non_blocking=True)
        self.saved[self.name_prefix + name] = host
    return t

  def reuse(self, name: str):
    """In the recompute forward: the kept tensor for `name`, or None if it must be recomputed."""
    if self.recompute and self.saved is not None and (self.name_prefix + name) in self.saved:
      t = self.saved[self.name_prefix + name]
      if t.device.type == "cpu" and self.positions.is_cuda:
        t = t.to(self.positions.device, non_blocking=True)
      return t
    return None
