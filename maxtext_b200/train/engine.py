"""Hand-scheduled training step.

Where MaxText traces `train_step` once and lets XLA schedule the collectives
(src/maxtext/trainers/pre_train/train.py:422-746; FSDP all-gather / reduce-scatter are implicit,
overlap comes from the latency-hiding scheduler flags in src/maxtext/configs/gpu/a3/llama_2_7b/1vm.sh),
this engine runs the model unit by unit with an explicit schedule:

  forward   : [prefetch gather(u+1)] -> no-grad forward(u), keep the layer input (+ the tensors named by
              remat_policy) -> release(u)
  head      : fused output projection + cross entropy computes the loss AND d(hidden) in one pass
  backward  : [prefetch gather(u-1)] -> recompute forward(u) with autograd -> backward -> dW lands in the
              fp32 gradient buffer of the unit -> async reduce-scatter(u) -> release(u)
  update    : global grad norm (one scalar all-reduce) -> clip factor and 1/total_weights stay on the
              device -> single fused AdamW launch over the local flat shard

The same code path serves one GPU (nothing to gather) and any FSDP/DP layout of the mesh. The
step-wise API (`fwd_bwd` may be called several times before `update`) matches
src/maxtext/training_engine/maxtext_engine.py:333-384 and implements gradient accumulation with
token-weighted normalisation (src/maxtext/utils/gradient_accumulation.py:110-190).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..models.transformer import Transformer
from ..layers.blocks import sp_enabled as L_sp_enabled
from ..ops import functional as F
from ..optimizers import factory as opt_factory
from ..optimizers.schedules import make_schedule

EPS = 1e-8


class TrainEngine:
  def __init__(self, config, mesh=None, device=None, model: Transformer | None = None, init: bool = True):
    self.config = c = config
    self.mesh = mesh
    if device is None:
      device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and c.hardware != "cpu" \
          else torch.device("cpu")
    self.device = torch.device(device)
    if mesh is not None and L_sp_enabled(c) and mesh.axis_size(("tensor", "tensor_sequence")) > 1:
      # the sequence-split residual stream is implemented for the plain layer loop only; a silent fallback would leave the
      # norm-scale gradients flagged as partial sums although they are complete
      if mesh.axis_size(("context", "context_usp_ulysses")) > 1 or mesh.axis_size("stage") > 1:
        raise NotImplementedError("tensor_sequence parallelism cannot be combined with context or pipeline parallelism yet")
      if int(getattr(c, "mtp_num_layers", 0) or 0) > 0:
        raise NotImplementedError("multi-token prediction is not implemented under tensor_sequence parallelism")
    if str(getattr(c, "attention_type", "global")) == "block_diffusion":
      if str(getattr(c, "training_objective", "causal_lm")) != "block_diffusion":
        # src/maxtext/trainers/pre_train/train.py:115-119: next-token labels would leak inside a bidirectional block
        raise ValueError("block-diffusion attention requires training_objective=block_diffusion")
      if mesh is not None and mesh.axis_size(("context", "context_usp_ulysses")) > 1:
        raise NotImplementedError("block-diffusion attention is not implemented under context parallelism")
    self.model = model or Transformer(c, mesh, self.device)
    from ..ops import quantization as _quant
    _quant.set_mode(str(c.quantization or ""))
    _quant.set_delayed_scaling(int(getattr(c, "fp8_amax_history_len", 0)))
    _quant.set_block_scaling(bool(getattr(c, "fp8_block_scaling", False)))
    self.store = self.model.store
    if init:
      self.store.initialize(seed=c.init_weights_seed)
    self.schedule = make_schedule(c)
    self.optimizer = opt_factory.make_optimizer(c, self.store, self.model)
    self.step_count = 0
    self.world = mesh.world if mesh is not None else 1
    # DiLoCo: a replica (all axes but `diloco`) is a self-contained training job; losses, norms and gradients stay inside it
    n_rep = mesh.axis_size("diloco") if mesh is not None else 1
    self.inner_group = mesh.group(tuple(a for a in mesh.axis_names if a != "diloco")) if n_rep > 1 else None
    self.inner_world = self.world // n_rep
    self._accum = None
    self._units = self._ordered_units()
    from ..models import families as _fam
    # all MoE blocks of the model, also those that live on other pipeline stages (the balance loss is averaged over them)
    self.n_moe_layers = sum(1 for pl in _fam.layer_plans(c) for b in pl.blocks if b.mlp in ("moe", "moe_shared"))
    self.all_group = None  # WORLD

  # ------------------------------------------------------------------ unit bookkeeping
  def _ordered_units(self):
    """Store units in execution order: embed*, layer_i*, head* (a logical unit may be split by shard group)."""
    order = []
    for name in self.model.units_in_order():
      order.append([u for k, u in self.store.units.items() if k == name or k.startswith(name + "#")])
    return order

  def _gather(self, idx, async_op=True):
    if 0 <= idx < len(self._units):
      for u in self._units[idx]:
        if u.group_size > 1 and not u.resident:
          u._work = self.store.gather_unit(u, async_op=async_op)

  def _wait_gather(self, idx):
    for u in self._units[idx]:
      w = getattr(u, "_work", None)
      if w is not None:
        w.wait()
        u._work = None

  def _release(self, idx):
    for u in self._units[idx]:
      self.store.release_full(u)

  def _shard_for_context(self, batch: dict) -> dict:
    """Context parallelism: every rank of a context group reads the same rows and keeps its slice of the sequence."""
    if self.mesh is None:
      return batch
    axes = ("context", "context_usp_ulysses")
    cp = self.mesh.axis_size(axes)
    if cp == 1:
      return batch
    from ..parallel.context_parallel import shard_batch
    return shard_batch(batch, self.mesh.axis_index(axes), cp, bool(self.config.context_parallel_load_balance))

  # ------------------------------------------------------------------ forward + backward
  def fwd_bwd(self, batch: dict, compute_grads: bool = True) -> dict:
    """Accumulates gradients of sum_t w_t * loss_t (+ scaled aux losses) into the gradient shards.

    batch: inputs, targets [B,S] int; inputs_position, inputs_segmentation, targets_segmentation optional.
    """
    c, model, store = self.config, self.model, self.store
    batch = self._shard_for_context(batch)
    tokens = batch["inputs"].to(self.device, non_blocking=True)
    targets = batch["targets"].to(self.device, non_blocking=True)
    B, S = tokens.shape
    positions = batch.get("inputs_position")
    positions = positions.to(self.device, non_blocking=True) if positions is not None else \
        torch.arange(S, device=self.device, dtype=torch.int32)[None].expand(B, S)
    seg = batch.get("inputs_segmentation")
    seg = seg.to(self.device, non_blocking=True) if seg is not None else None
    tseg = batch.get("targets_segmentation")
    weights = (tseg.to(self.device) != 0).float() if tseg is not None else torch.ones(B, S, device=self.device)
    if batch.get("loss_weights") is not None:
      # post-training objectives (DPO, GRPO...) express their gradient as per-token weights on the token losses
      weights = batch["loss_weights"].to(self.device).float()
    if c.dataset_type == "synthetic" and not c.packing_in_synthetic:
      seg = None   # synthetic batches are one segment per row by construction: skip the mask work
    diffusion = str(getattr(c, "training_objective", "causal_lm")) == "block_diffusion"
    bd_index = None
    if diffusion:
      # block diffusion (src/maxtext/trainers/pre_train/train.py:114-142,201-228): the batch names its own targets
      for k in ("corruption_mask", "targets_loss_mask"):
        if batch.get(k) is None or tuple(batch[k].shape) != (B, S):
          raise ValueError(f"block-diffusion loss needs the batch mask {k!r} with the shape of targets")
      weights = weights * (batch["targets_loss_mask"].to(self.device) != 0).float()
      from ..diffusion.block_diffusion import source_indices
      tpos = batch.get("targets_position", batch.get("inputs_position"))
      bd_index = source_indices(str(c.block_diffusion_logit_alignment), S, tpos.to(self.device) if tpos is not None else None,
                                (tseg.to(self.device) != 0) if tseg is not None else None, B, self.device)

    first_micro = self._accum is None
    if first_micro:
      self._accum = dict(loss_sum=torch.zeros((), device=self.device), z_sum=torch.zeros((), device=self.device),
                         weights=torch.zeros((), device=self.device), aux=torch.zeros((), device=self.device), micro=0)
      if compute_grads:
        store.begin_step()
    acc = self._accum
    acc["micro"] += 1
    accumulate_rs = compute_grads and not first_micro

    n_units = len(self._units)
    ctx = model.make_ctx(positions, seg, "train", tokens)
    if bool(getattr(c, "use_batch_split_schedule", False)):
      ctx.batch_split = max(2, int(getattr(c, "batch_split_factor", 1) or 1))
    if str(getattr(c, "attention_type", "global")) == "block_diffusion":
      from ..diffusion.block_diffusion import same_block_mask
      ctx.bidir = same_block_mask(positions, int(c.causal_block_size), seg)
    p3 = batch.get("inputs_position3")          # [B, S, 3] multi-axis rotary positions of multimodal rows (`use_mrope`)
    ctx.positions3 = p3.to(self.device) if p3 is not None else None
    if float(c.dropout_rate) > 0 and bool(c.enable_dropout) and compute_grads:
      # one seed per micro-batch and data shard; tensor ranks of a shard share it (they hold the same activations)
      shard = self.mesh.axis_index(("data", "fsdp", "fsdp_transpose", "expert", "context", "context_usp_ulysses")) if self.mesh is not None else 0
      ctx.dropout_seed = (int(c.init_weights_seed) * 7919 + self.step_count * 613 + acc["micro"]) * 4099 + shard
    if c.use_qk_clip:
      self._max_logits = getattr(self, "_max_logits", None) or {}
      ctx.max_logits = self._max_logits
    if c.routed_bias and c.routed_bias_update_rate > 0:
      self._expert_counts = getattr(self, "_expert_counts", None) or {}
      ctx.expert_counts = self._expert_counts
    # ---- forward
    self._gather(0, async_op=False)
    self._gather(1)
    mm = self._encode_images(batch, tokens, ctx)
    am = self._encode_audio(batch)
    if am is not None:
      mm = am if mm is None else [mm, am]
    x = self._run_embed(tokens, positions, grad=False, mm=mm)
    # tensor-sequence parallelism: between blocks every tensor rank holds its part of the sequence only
    sp_on = ctx.tp_size > 1 and L_sp_enabled(c) and ctx.cp_size == 1
    if sp_on:
      from ..parallel import sequence_parallel as sp
      assert S % ctx.tp_size == 0, "the sequence must divide by the tensor-sequence degree"
      ctx.sp = True
      x = sp.local_seq(x, ctx.tp_group)
    self._release(0) if self._units[0] and self._units[0][0].group_size > 1 and not c.logits_via_embedding else None
    ckpts = []
    for i, layer in enumerate(model.layers):
      ui = i + 1
      self._wait_gather(ui)
      self._gather(ui + 1)
      saved = {}
      ctx.saved, ctx.recompute, ctx.layer_index, ctx.aux_losses = saved, False, i, []
      with torch.no_grad():
        y = layer(x, ctx)
      aux_val = sum(a for _, a in ctx.aux_losses) if ctx.aux_losses else None
      if aux_val is not None:
        acc["aux"] += aux_val.detach().float()
      ckpts.append((x, saved))
      x = y
      if not (i == len(model.layers) - 1):
        self._release(ui)
    # ---- head: loss and d(hidden) in one pass
    hi = n_units - 1
    self._gather(hi)                 # a no-op when the prefetch above already covered it
    self._wait_gather(hi)
    if c.logits_via_embedding:
      self._gather(0, async_op=False)
    w_flat = weights.reshape(-1)
    total_w = w_flat.sum() if batch.get("loss_normalizer") is None else \
        torch.as_tensor(float(batch["loss_normalizer"]), device=self.device, dtype=torch.float32)
    head_units = self._units[hi] + (self._units[0] if c.logits_via_embedding else [])
    if compute_grads:
      for u in head_units:
        store.acquire_full_grad(u)
    if sp_on:
      x = sp.all_gather_seq(x, ctx.tp_group)               # the head scores every token on every tensor rank, as without SP
    if bd_index is not None:
      # shifted alignment: target s is scored by the state of the slot holding the previous position
      gi = bd_index[:, :, None].expand(B, S, x.shape[-1])
      loss_sum, z_sum, dxa = self._run_head(x.gather(1, gi), targets.reshape(-1), w_flat, compute_grads)
      dx = torch.zeros_like(x).scatter_add_(1, gi, dxa.view(B, S, -1)).view(dxa.shape) if dxa is not None else None
    else:
      loss_sum, z_sum, dx = self._run_head(x, targets.reshape(-1), w_flat, compute_grads)
    if sp_on and dx is not None:
      dx = sp.local_seq(dx.view(B, S, -1), ctx.tp_group)
    acc["loss_sum"] += loss_sum
    acc["z_sum"] += z_sum
    acc["weights"] += total_w
    mtp_embed_grads = []
    if model.mtp_layers and compute_grads:
      dx, mtp_embed_grads = self._run_mtp(x, dx, tokens, targets, weights, positions, seg, total_w, acc, ctx, accumulate_rs)
    if not compute_grads:
      for i in range(n_units):
        self._release(i)
      return acc
    self._finish_unit_grads(hi, accumulate_rs, skip_embed=True)
    self._release(hi)
    # ---- backward through the layers
    aux_scale = None
    if self.n_moe_layers and c.load_balance_loss_weight > 0:
      # the update divides every gradient by the global token weight; the balance loss is a mean over each rank's own rows,
      # and the ranks' gradients are summed, so it is seeded with weight / (layers x data shards)
      aux_scale = self._global_weight(total_w) / self.n_moe_layers / self._data_shards()
    self._gather(len(model.layers) - 1)  # unit index of layer L-2 is L-1
    train_towers = mm is not None and not bool(getattr(c, "freeze_vision_encoder_params", True))
    deep_grads: dict = {}
    for i in reversed(range(len(model.layers))):
      ui = i + 1
      layer = model.layers[i]
      self._wait_gather(ui)
      self._gather(ui - 1)
      for u in self._units[ui]:
        store.acquire_full_grad(u)
      x_in, saved = ckpts.pop()
      x_in = x_in.detach().requires_grad_(True)
      ctx.saved, ctx.recompute, ctx.layer_index, ctx.aux_losses = saved, True, i, []
      deep_leaf = None
      if train_towers and ctx.deepstack is not None and layer.index < len(ctx.deepstack[1]):
        # a trainable tower also feeds this layer directly (deepstack): differentiate with respect to that feature as well
        deep_leaf = ctx.deepstack[1][layer.index].detach().requires_grad_(True)
        feats = list(ctx.deepstack[1])
        feats[layer.index] = deep_leaf
        ctx.deepstack = (ctx.deepstack[0], feats)
      with torch.enable_grad():
        y = layer(x_in, ctx)
        outs, grads = [y], [dx]
        if aux_scale is not None and ctx.aux_losses:
          for _, a in ctx.aux_losses:
            outs.append(a)
            grads.append(aux_scale.to(a.dtype))
      torch.autograd.backward(outs, grads)
      dx = x_in.grad
      if deep_leaf is not None and deep_leaf.grad is not None:
        deep_grads[layer.index] = deep_leaf.grad
      del y, outs, grads, x_in, saved
      for p in layer.params:
        p.collect_leaf_grad()
      self._finish_unit_grads(ui, accumulate_rs)
      self._release(ui)
    # ---- embedding backward
    self._wait_gather(0)
    emb_units = self._units[0]
    if not c.logits_via_embedding:
      for u in emb_units:
        store.acquire_full_grad(u)
    if sp_on:
      dx = sp.all_gather_seq(dx, ctx.tp_group)
    if mm is not None and not bool(getattr(c, "freeze_vision_encoder_params", True)):
      self._towers_backward(batch, tokens, positions, dx, accumulate_rs, deep_grads)
    else:
      self._run_embed(tokens, positions, grad=True, dx=dx, mm=mm)
    for r_tokens, r_pos, d_emb in mtp_embed_grads:          # embeddings of the tokens further ahead, used by the MTP modules
      self._run_embed(r_tokens, r_pos, grad=True, dx=d_emb)
    self._finish_unit_grads(0, accumulate_rs)
    self._release(0)
    store.wait_reduce_scatters()
    return acc

  def _run_mtp(self, x, dx_main, tokens, targets, weights, positions, seg, total_w, acc, ctx, accumulate_rs):
    """Multi-token prediction (src/maxtext/layers/multi_token_prediction.py:334-531): module k predicts the token k + 1
    steps ahead from the previous module's hidden state and the embedding of the token k steps ahead, through the shared
    output head. loss = mtp_loss_scaling_factor * sum_k sum(xent_k * mask_k) / sum_k sum(mask_k), added to the main loss.
    Returns d(final hidden) including the MTP paths, and the deferred embedding gradients."""
    from ..models.transformer import roll_left
    c, model, store = self.config, self.model, self.store
    mi = len(self._units) - 2
    self._gather(mi, async_op=False)
    self._wait_gather(mi)
    self._gather(0, async_op=False)          # the modules embed the tokens further ahead with the shared table
    for u in self._units[mi]:
      store.acquire_full_grad(u)
    B, S = tokens.shape
    r_tok, r_tgt, r_w, r_pos, r_seg = tokens, targets, weights, positions, seg
    rolled = []
    for _ in model.mtp_layers:
      r_tok, r_tgt, r_w, r_pos = (roll_left(t, r_seg) for t in (r_tok, r_tgt, r_w, r_pos))
      r_seg = roll_left(r_seg) if r_seg is not None else None
      rolled.append((r_tok, r_tgt, r_w, r_pos))
    mtp_w = sum(w.sum() for _, _, w, _ in rolled)
    # token losses are summed un-normalised and divided by the main total weight in the optimizer; rescale so that the
    # MTP term ends up divided by its own weight and multiplied by the scaling factor
    factor = float(c.mtp_loss_scaling_factor) * self._global_weight(total_w) / (self._global_weight(mtp_w) + EPS)
    x_in = x.detach().requires_grad_(True)
    h, outs, grads, embs = x_in, [], [], []
    ctx.saved, ctx.recompute, ctx.aux_losses = {}, False, []
    mtp_loss = torch.zeros((), device=self.device)
    with torch.enable_grad():
      for layer, (tk, tg, w, ps) in zip(model.mtp_layers, rolled):
        with torch.no_grad():
          e = model.embed(tk, ps)
        e = e.detach().requires_grad_(True)
        embs.append((tk, ps, e))
        h = layer(h, e, ctx)
        loss_k, _, dh = self._run_head(h, tg.reshape(-1), (w * factor).reshape(-1), True)
        mtp_loss = mtp_loss + loss_k
        outs.append(h)
        grads.append(dh)
    torch.autograd.backward(outs, grads)
    for p in model.mtp_params:
      p.collect_leaf_grad()
    self._finish_unit_grads(mi, accumulate_rs)
    self._release(mi)
    acc["mtp"] = acc.get("mtp", torch.zeros((), device=self.device)) + mtp_loss
    return dx_main + x_in.grad, [(tk, ps, e.grad) for tk, ps, e in embs]

  def _global_weight(self, total_w):
    """Token weight of the whole (inner) job, every token counted once."""
    if self.inner_world > 1:
      t = total_w.clone()
      dist.all_reduce(t, group=self.inner_group)
      # tensor ranks and pipeline stages see the same tokens
      dup = self.mesh.axis_size(("tensor", "tensor_sequence", "stage")) if self.mesh is not None else 1
      return t / dup if dup > 1 else t
    return total_w

  def _data_shards(self) -> int:
    """Ranks of the (inner) job that see different tokens: the product of the batch and sequence axes."""
    if self.mesh is None:
      return 1
    return max(1, self.mesh.axis_size(("data", "fsdp", "fsdp_transpose", "expert", "context", "context_usp_ulysses")))

  def _encode_images(self, batch: dict, tokens, ctx):
    """Multimodal batches (`images` [B, N, 3, H, W] + `image_mask` [B, S]): run the frozen vision tower once, without
    gradient, and let the tokens of each image attend to each other in both directions."""
    if batch.get("images") is None or self.model.vision is None:
      return None
    from ..multimodal.utils import bidirectional_block_mask
    units = [u for k, u in self.store.units.items() if k == "vision" or k.startswith("vision#")]
    for u in units:
      if u.group_size > 1 and not u.resident:
        self.store.gather_unit(u, async_op=False)
    with torch.no_grad():
      mm = self.model.encode_images(batch["images"].to(self.device), batch["image_mask"].to(self.device))
    for u in units:
      self.store.release_full(u)
    ctx.deepstack = getattr(self.model, "_deepstack", None)
    if self.model.vision.__class__.__name__ in ("Gemma3Vision", "Gemma4Vision"):    # Llama-4 keeps plain causal attention over image tokens
      ctx.bidir = bidirectional_block_mask(mm[1])
    return mm

  def _encode_audio(self, batch: dict):
    """Batches with `audio` ([B, mel, frames] or a list of clips) + `audio_mask` [B, S]: run the frozen audio tower once."""
    if batch.get("audio") is None or self.model.audio is None:
      return None
    units = [u for k, u in self.store.units.items() if k == "audio" or k.startswith("audio#")]
    for u in units:
      if u.group_size > 1 and not u.resident:
        self.store.gather_unit(u, async_op=False)
    with torch.no_grad():
      am = self.model.encode_audio(batch["audio"], batch["audio_mask"].to(self.device))
    for u in units:
      self.store.release_full(u)
    return am

  def _towers_backward(self, batch, tokens, positions, dx, accumulate_rs, deep_grads=None):
    """`freeze_vision_encoder_params=false`: the towers ran without gradient in the forward pass; here they run again under
    autograd, the soft tokens enter the embedding, and d(embedding output) flows back into the tower parameters together with
    the embedding table's own gradient. Features that reach the decoder by another route (Qwen3-VL deepstack, added after the
    first layers) bring the gradients collected while those layers were replayed (`deep_grads`: feature index -> gradient)."""
    model, store = self.model, self.store
    units = [u for k, u in store.units.items() if k.split("#")[0] in ("vision", "audio")]
    for u in units:
      if u.group_size > 1 and not u.resident:
        store.gather_unit(u, async_op=False)
      store.acquire_full_grad(u)
    with torch.enable_grad():
      mm_g = []
      if batch.get("images") is not None and model.vision is not None:
        mm_g.append(model.encode_images(batch["images"].to(self.device), batch["image_mask"].to(self.device)))
      if batch.get("audio") is not None and model.audio is not None:
        mm_g.append(model.encode_audio(batch["audio"], batch["audio_mask"].to(self.device)))
      x = model.embed(tokens, positions, mm_g[0] if len(mm_g) == 1 else mm_g)
      outs, grads = [x], [dx]
      deep = getattr(model, "_deepstack", None)
      for i, g in (deep_grads or {}).items():
        if deep is not None and i < len(deep[1]) and deep[1][i].requires_grad:
          outs.append(deep[1][i])
          grads.append(g.to(deep[1][i].dtype).reshape(deep[1][i].shape))
    torch.autograd.backward(outs, grads)
    for p in list(model.embed_params) + list(model.vision_params) + list(model.audio_params):
      p.collect_leaf_grad()
    for u in units:
      if u.group_size > 1:
        store.reduce_scatter_unit(u, async_op=True, accumulate=accumulate_rs)
      store.release_full(u)

  def _run_embed(self, tokens, positions, grad: bool, dx=None, mm=None):
    model = self.model
    if not grad:
      with torch.no_grad():
        return model.embed(tokens, positions, mm)
    with torch.enable_grad():
      x = model.embed(tokens, positions, mm)
    torch.autograd.backward([x], [dx])
    for p in model.embed_params:
      p.collect_leaf_grad()
    return None

  def custom_loss_step(self, batch: dict, loss_fn) -> dict:
    """One optimizer step on loss_fn(logits [T,V] fp32, targets [T], mask [T]) -> scalar, differentiated by autograd
    through the output head (full logits are materialised: meant for small models, e.g. distillation)."""
    self._custom_loss = loss_fn
    try:
      b = dict(batch)
      b["loss_normalizer"] = 1.0
      self.fwd_bwd(b)
    finally:
      self._custom_loss = None
    return self.update()

  def _run_head(self, x, targets, weights, compute_grads):
    c, model = self.config, self.model
    B, S, D = x.shape[0], x.shape[1], x.shape[-1]      # x is [B, S, k, D] when hyper-connections widen the residual stream
    fn = getattr(self, "_custom_loss", None)
    if fn is not None and compute_grads:
      x_in = x.detach().requires_grad_(True)
      with torch.enable_grad():
        h = model.final_norm(x_in)
        logits = F.linear(h.reshape(B * S, D), model.head_param()).float() * model.head_logit_scale()
        loss = fn(logits, targets.long(), weights)
      loss.backward()
      for p in model.head_params:
        p.collect_leaf_grad()
      return loss.detach().float(), torch.zeros((), device=self.device), x_in.grad
    x_in = x.detach().requires_grad_(compute_grads)
    with torch.set_grad_enabled(compute_grads):
      h = model.final_norm(x_in)
    chunk = max(256, (B * S) // max(1, c.num_vocab_tiling)) if c.num_vocab_tiling > 1 else min(B * S, 2048)
    loss_sum, z_sum, dh = F.fused_head_loss(h.detach().reshape(B * S, D), model.head_param(), targets, weights,
                                            c.z_loss_multiplier, c.final_logits_soft_cap, chunk, model.head_logit_scale(),
                                            compute_grads)
    dx = None
    if compute_grads:
      torch.autograd.backward([h], [dh.view(B, S, D)])
      dx = x_in.grad
      for p in model.head_params:
        p.collect_leaf_grad()
    return loss_sum, z_sum, dx

  def _finish_unit_grads(self, idx, accumulate, skip_embed=False):
    """Launch the reduce-scatter (and replica all-reduce) of every store unit behind schedule slot `idx`."""
    store = self.store
    units = list(self._units[idx])
    if idx == len(self._units) - 1 and self.config.logits_via_embedding and not skip_embed:
      pass
    for u in units:
      if u.group_size > 1:
        store.reduce_scatter_unit(u, async_op=True, accumulate=accumulate)

  # ------------------------------------------------------------------ update
  def update(self) -> dict:
    """Normalise, clip, apply the optimizer; returns device-side metrics (no host sync here)."""
    c, store = self.config, self.store
    acc = self._accum
    assert acc is not None, "update() called before fwd_bwd()"
    self._accum = None
    store.finish_resident_grads()
    stats = torch.stack([acc["loss_sum"], acc["z_sum"], acc["weights"], acc["aux"], acc.get("mtp", torch.zeros((), device=self.device))])
    if self.inner_world > 1:
      dist.all_reduce(stats, group=self.inner_group)
      # the balance loss: summed over pipeline stages (each holds some of the layers), averaged over the ranks that hold the
      # same layers (data shards and tensor ranks)
      stats[3] /= max(1, self.inner_world // (self.mesh.axis_size("stage") if self.mesh is not None else 1))
      # ranks along the tensor axes score the same tokens: count each token once (the gradient itself is summed over the
      # data axes only, so without this the normaliser, and with it the clipping threshold, would be off by the TP degree)
      dup = self.mesh.axis_size(("tensor", "tensor_sequence")) if self.mesh is not None else 1
      if dup > 1:
        stats[[0, 1, 2, 4]] /= dup
    loss_sum, z_sum, total_w, aux, mtp_sum = stats[0], stats[1], stats[2], stats[3], stats[4]
    aux = aux / max(1, acc["micro"]) / max(1, self.n_moe_layers)
    inv_w = 1.0 / (total_w + EPS)
    # replica (data-parallel) gradient reduction for units replicated across batch axes
    self._reduce_replicas()
    raw_sq = self._grad_sumsq()
    raw_norm = torch.sqrt(raw_sq) * inv_w
    thr = float(c.gradient_clipping_threshold)
    if thr > 0:
      clip = torch.where(raw_norm < thr, torch.ones_like(raw_norm), thr / (raw_norm + 1e-30))
    else:
      clip = torch.ones_like(raw_norm)
    grad_scale = (clip * inv_w).reshape(1).float()
    lr = self.schedule(self.step_count)
    opt_metrics = self.optimizer.step(grad_scale, lr, self.step_count + 1, loss=(loss_sum * inv_w), grad_norm=raw_norm)
    self.step_count += 1
    if getattr(self, "_expert_counts", None):
      self._apply_routed_bias_update()
    if c.use_qk_clip and getattr(self, "_max_logits", None):
      opt_metrics = dict(opt_metrics)
      opt_metrics["learning/max_attention_logit"] = self._apply_qk_clip()
    if getattr(store, "fused", False):
      store.symm.barrier(0)       # updated shards are final on every rank before the next step reads them over NVLink
    lm_loss = loss_sum * inv_w
    metrics = {
        "learning/loss": lm_loss + aux + mtp_sum * inv_w, "learning/lm_loss": lm_loss, "learning/mtp_loss": mtp_sum * inv_w,
        "learning/z_loss": z_sum * inv_w,
        "learning/moe_lb_loss": aux, "learning/total_weights": total_w, "learning/raw_grad_norm": raw_norm,
        "learning/grad_norm": raw_norm * clip, "learning/current_learning_rate": torch.tensor(lr),
    }
    metrics.update(opt_metrics)
    return metrics

  @torch.no_grad()
  def _apply_routed_bias_update(self):
    """Auxiliary-loss-free load balancing (DeepSeek-V3; src/maxtext/layers/moe.py:215-236, train.py:646-690): after the
    optimizer step every routed expert's selection bias moves by +rate if it received fewer tokens than average this step
    and by -rate if it received more."""
    c, store = self.config, self.store
    rate = float(c.routed_bias_update_rate)
    for moe, cnt in self._expert_counts.items():
      if self.inner_world > 1:
        dist.all_reduce(cnt, group=self.inner_group)
      delta = torch.sign(cnt.sum() / cnt.numel() - cnt) * rate
      p = moe.gate_bias
      u = store.unit_of(p)
      off = u.offsets[u.params.index(p)]
      lo, hi = u.group_rank * u.chunk, (u.group_rank + 1) * u.chunk
      a, b = max(off, lo), min(off + p.pdef.numel, hi)
      if a < b:
        store.shard_view(u, store.master)[a - lo: b - lo].add_(delta[a - off: b - off].to(store.master.dtype))
    store.sync_compute_from_master()
    self._expert_counts.clear()

  @torch.no_grad()
  def _apply_qk_clip(self):
    """QK-clip (MuonClip; src/maxtext/utils/qk_clip_utils.py:86-136): after the update, every MLA head whose largest
    attention logit exceeded qk_clip_threshold has its query / key weights shrunk by gamma = tau / s_max: the no-position
    parts of wq_b and wkv_b by sqrt(gamma) each, the rotary part of wq_b by gamma (the rotary key is shared by all heads)."""
    c, store = self.config, self.store
    tau = float(c.qk_clip_threshold)
    overall = torch.zeros((), device=self.device)
    for (_, mla), smax in self._max_logits.items():
      if self.inner_world > 1:
        dist.all_reduce(smax, op=dist.ReduceOp.MAX, group=self.inner_group)
      overall = torch.maximum(overall, smax.max())
      gamma = torch.clamp(tau / (smax + 1e-6), max=1.0)                        # [heads on this rank]
      rt = torch.sqrt(gamma)
      q_rows = torch.cat([rt[:, None].expand(-1, mla.nope), gamma[:, None].expand(-1, mla.rope_d)], 1).reshape(-1)
      kv_rows = torch.cat([rt[:, None].expand(-1, mla.nope), torch.ones_like(rt)[:, None].expand(-1, mla.vd)], 1).reshape(-1)
      wq = mla.wq_b if mla.query is None else mla.query
      for p, rows in ((wq, q_rows), (mla.wkv_b, kv_rows)):
        u = store.unit_of(p)
        off = u.offsets[u.params.index(p)]
        lo, hi = u.group_rank * u.chunk, (u.group_rank + 1) * u.chunk
        a, b = max(off, lo), min(off + p.pdef.numel, hi)
        if a < b:
          n_in = p.pdef.shape[1]
          idx = torch.arange(a - off, b - off, device=self.device) // n_in          # internal layout [out rows, in]
          store.shard_view(u, store.master)[a - lo: b - lo].mul_(rows[idx].to(store.master.dtype))
    store.sync_compute_from_master()
    self._max_logits.clear()
    return overall

  def _reduce_replicas(self):
    store, mesh = self.store, self.mesh
    if mesh is None or self.inner_world == 1:
      return
    for u in store.units.values():
      per_param = [store.replica_axes(u, [p]) for p in u.params]
      if len(set(per_param)) > 1:
        # an unsharded unit that mixes tensors split over a batch axis (experts over `expert`) with replicated ones (norm
        # scales): reduce each tensor over the axes it is replicated on
        assert u.group_size == 1, "mixed replication is only laid out in unsharded units"
        for p, off, axes in zip(u.params, u.offsets, per_param):
          g = mesh.group(axes) if axes else None
          if g is not None:
            a = u.shard_offset + off
            dist.all_reduce(store.grad_shard[a: a + p.pdef.numel], group=g)
        continue
      axes = per_param[0] if per_param else ()
      if axes:
        g = mesh.group(axes)
        if g is not None:
          dist.all_reduce(store.shard_view(u, store.grad_shard), group=g)
    tp_axes = ("tensor", "tensor_sequence")
    if mesh.axis_size(tp_axes) > 1:
      # parameters every tensor rank holds whole but applies to its own heads only (per-head q/k norm scales)
      tg = mesh.group(tp_axes)
      for u in store.units.values():
        for p, off in zip(u.params, u.offsets):
          if p.pdef.tp_partial and not p.pdef.frozen:
            # the part of this tensor that lies in this rank's shard of the unit (all of it when the unit is not sharded); the
            # tensor ranks that share a shard index hold the same part
            lo_ = u.group_rank * u.chunk if u.group_size > 1 else 0
            hi_ = lo_ + (u.chunk if u.group_size > 1 else u.numel)
            s0, s1 = max(off, lo_), min(off + p.pdef.numel, hi_)
            if s1 > s0:
              a = u.shard_offset + (s0 - lo_)
              dist.all_reduce(store.grad_shard[a: a + (s1 - s0)], group=tg)

  def _grad_sumsq(self):
    """Sum of squares of the (un-normalised) global gradient: local shards, de-duplicated, all-reduced."""
    store = self.store
    if self.inner_world == 1:
      return F.sum_of_squares(store.grad_shard)
    total = torch.zeros((), dtype=torch.float32, device=self.device)
    fused_sq = getattr(store, "fused", False) and store.gradsq_valid
    if fused_sq:
      total = total + store.gradsq[0]      # partials emitted by the fused reduce-scatter kernels
    for u in store.units.values():
      if fused_sq and u.group_size > 1:
        continue
      if len({(p.pdef.tp_dim is None, p.pdef.ep_dim is None) for p in u.params}) > 1:
        # a unit that holds both split and replicated tensors (e.g. attention kernels next to the router): weigh the part
        # of each tensor that lies in this rank's shard by that tensor's own multiplicity
        lo = u.group_rank * u.chunk if u.group_size > 1 else 0
        hi = lo + (u.chunk if u.group_size > 1 else u.numel)
        for p, off in zip(u.params, u.offsets):
          a, b = max(off, lo), min(off + p.pdef.numel, hi)
          if a < b:
            piece = store.grad_shard[u.shard_offset + a - lo: u.shard_offset + b - lo]
            total = total + F.sum_of_squares(piece) / self._replication(u, [p])
        continue
      sq = F.sum_of_squares(store.shard_view(u, store.grad_shard))
      total = total + sq / self._replication(u)
    dist.all_reduce(total, group=self.inner_group)
    return total

  def _replication(self, u, params=None) -> float:
    """How many ranks hold an identical copy of this unit's gradient shard (or of the given tensors of it)."""
    mesh = self.mesh
    params = u.params if params is None else params
    distinct = u.group_size
    tp = mesh.axis_size(("tensor", "tensor_sequence"))
    if tp > 1 and any(p.pdef.tp_dim is not None for p in params):
      distinct *= tp
    ep = mesh.axis_size("expert")
    if ep > 1 and any(p.pdef.ep_dim is not None for p in params):
      distinct *= ep
    return max(1.0, self.inner_world / distinct)

  def train_step(self, batch: dict) -> dict:
    """One optimizer step over `gradient_accumulation_steps` micro-batches split along the batch dim."""
    g = int(self.config.gradient_accumulation_steps)
    if g == 1:
      self.fwd_bwd(batch)
    else:
      B = batch["inputs"].shape[0]
      assert B % g == 0, "batch must divide by gradient_accumulation_steps"
      mb = B // g
      for k in range(g):
        self.fwd_bwd({key: v[k * mb:(k + 1) * mb] for key, v in batch.items()})
    return self.update()

  @torch.no_grad()
  def token_losses(self, batch: dict) -> torch.Tensor:
    """Per-token cross entropy [B, S] (no gradients): the building block of sequence log-probabilities."""
    model = self.model
    batch = self._shard_for_context(batch)
    tokens = batch["inputs"].to(self.device)
    targets = batch["targets"].to(self.device)
    B, S = tokens.shape
    positions = batch.get("inputs_position")
    positions = positions.to(self.device) if positions is not None else torch.arange(S, device=self.device)[None].expand(B, S)
    seg = batch.get("inputs_segmentation")
    seg = seg.to(self.device) if seg is not None else None
    ctx = model.make_ctx(positions, seg, "train", tokens)
    p3 = batch.get("inputs_position3")          # [B, S, 3] multi-axis rotary positions of multimodal rows (`use_mrope`)
    ctx.positions3 = p3.to(self.device) if p3 is not None else None
    for i in range(len(self._units)):
      self._gather(i, async_op=False)
    x = model.embed(tokens, positions)
    for i, layer in enumerate(model.layers):
      ctx.layer_index, ctx.saved, ctx.aux_losses = i, None, []
      x = layer(x, ctx)
    h = model.final_norm(x).reshape(B * S, -1)
    out = torch.empty(B * S, dtype=torch.float32, device=self.device)
    from ..ops import reference as _ref
    for s0 in range(0, B * S, 2048):
      lg = F.head_logits(h[s0:s0 + 2048], model.head_param(), self.config.final_logits_soft_cap, model.head_logit_scale())
      out[s0:s0 + 2048] = _ref.cross_entropy(lg, targets.reshape(-1)[s0:s0 + 2048])[0]
    for i in range(len(self._units)):
      self._release(i)
    return out.view(B, S)

  @torch.no_grad()
  def eval_step(self, batch: dict) -> dict:
    acc = self.fwd_bwd(batch, compute_grads=False)
    self._accum = None
    stats = torch.stack([acc["loss_sum"], acc["weights"]])
    if self.world > 1:
      dist.all_reduce(stats)
    return {"evaluation/total_loss": stats[0], "evaluation/total_weights": stats[1],
            "evaluation/loss": stats[0] / (stats[1] + EPS)}
