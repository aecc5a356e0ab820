"""Pipeline parallelism over the `stage` mesh axis: GPipe and circular (repeated) schedules.

The reference implements the pipeline as a scanned `Pipeline` module whose stage dimension is sharded over `stage` and
whose activations rotate with a collective permute every iteration (src/maxtext/layers/pipeline.py; derived settings in
src/maxtext/configs/types.py:3565-3659). With one process per GPU the same schedule is explicit message passing: each
stage owns its layers' parameters (and only those), activations move to the next stage with point-to-point sends, and
the loop below is the schedule.

  forward : for repeat r, micro-batch m: recv x (or embed on stage 0, r = 0) -> layers of chunk r (no autograd, keep
            the chunk's layer inputs) -> send to the next stage (the last stage feeds stage 0 for the next repeat)
  backward: the same walk in reverse; each chunk is recomputed under autograd from its saved inputs, exactly as the
            single-stage engine does per layer, and d(input) goes back to the previous stage.
Bubble fraction (P - 1) / (M * R + P - 1) for P stages, M micro-batches, R repeats. Gradients accumulate over the
micro-batches in the fp32 gradient store; the optimizer step, norm and clipping are those of the base engine (the
squared-norm all-reduce spans the stages, every stage contributing its own parameters once).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.transformer import Transformer
from .engine import TrainEngine


class PipelineEngine(TrainEngine):
  def __init__(self, config, mesh, device=None, init: bool = True):
    assert mesh is not None and mesh.axis_size("stage") > 1, "PipelineEngine needs a mesh with stage > 1"
    assert not config.logits_via_embedding, "tied embeddings would live on two stages"
    self.P = mesh.axis_size("stage")
    self.s = mesh.axis_index("stage")
    dev = torch.device(device) if device is not None else None
    if dev is None:
      dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and config.hardware != "cpu" else torch.device("cpu")
    model = Transformer(config, mesh, dev, stage=(self.s, self.P))
    super().__init__(config, mesh, dev, model=model, init=init)
    ranks = mesh.ranks_along(("stage",))
    self.next_rank = ranks[(self.s + 1) % self.P]
    self.prev_rank = ranks[(self.s - 1) % self.P]
    self.R = max(1, int(config.num_pipeline_repeats))
    self.M = int(config.num_pipeline_microbatches)
    lps = int(config.num_layers_per_pipeline_stage)
    # chunk r = the layers this stage runs in repeat r
    self.chunks = [[l for l in self.model.layers if (l.index // lps) // self.P == r] for r in range(self.R)]
    self._uidx = {name: i for i, name in enumerate(self.model.units_in_order())}
    self._pending = []
    # NCCL runs the point-to-point operations of one communicator in issue order on one stream per peer. In the circular
    # schedule a stage sends activations of later micro-batches forward while the wrap-around of earlier ones comes back from
    # the same peer, and the two sides issue those in different orders: on one communicator that dead-locks. Every directed
    # (source, destination) pair therefore gets a communicator of its own, separately for activations and for gradients.
    # The plain schedule (one repeat) only ever moves activations one way and gradients the other, in the same order on both
    # sides, and stays on the default group.
    self._p2p = {}
    if dist.is_initialized() and dist.get_backend() == "nccl" and self.R > 1:
      seen = set()
      for r in range(mesh.world):                                  # collective: every rank creates every group, in one order
        ring = tuple(mesh.ranks_along(("stage",), r))
        if ring in seen:
          continue
        seen.add(ring)
        for tag in ("act", "grad"):
          for i in range(len(ring)):
            src, dst = (ring[i], ring[(i + 1) % len(ring)]) if tag == "act" else (ring[(i + 1) % len(ring)], ring[i])
            g = dist.new_group([src, dst]) if src != dst else None
            if mesh.rank in (src, dst):
              self._p2p[(src, dst, tag)] = g

  # ---- plumbing
  def _replication(self, u, params=None) -> float:
    return max(1.0, super()._replication(u, params) / self.P)        # every stage holds different parameters

  def _send(self, t, dst, tag="act"):
    self._pending.append((dist.isend(t.contiguous(), dst, group=self._p2p.get((self.mesh.rank, dst, tag))), t))

  def _recv(self, shape, dtype, src, tag="act"):
    buf = torch.empty(shape, dtype=dtype, device=self.device)
    dist.recv(buf, src, group=self._p2p.get((src, self.mesh.rank, tag)))
    return buf

  def _drain(self):
    for w, _ in self._pending:
      w.wait()
    self._pending = []

  def _has_prev(self, r):   # does chunk r on this stage take its input from another stage?
    return not (self.s == 0 and r == 0)

  def _has_next(self, r):
    return not (self.s == self.P - 1 and r == self.R - 1)

  # ---- schedule
  def fwd_bwd(self, batch: dict, compute_grads: bool = True) -> dict:
    c, model, store = self.config, self.model, self.store
    tokens = batch["inputs"].to(self.device)
    targets = batch["targets"].to(self.device)
    B, S = tokens.shape
    M = self.M
    assert B % M == 0, f"batch {B} must divide by num_pipeline_microbatches {M}"
    mb = B // M
    positions = batch.get("inputs_position")
    positions = positions.to(self.device) if positions is not None else \
        torch.arange(S, device=self.device, dtype=torch.int32)[None].expand(B, S)
    seg = batch.get("inputs_segmentation")
    seg = seg.to(self.device) if seg is not None else None
    tseg = batch.get("targets_segmentation")
    weights = (tseg.to(self.device) != 0).float() if tseg is not None else torch.ones(B, S, device=self.device)
    if c.dataset_type == "synthetic" and not c.packing_in_synthetic:
      seg = None
    first = self._accum is None
    if first:
      z = lambda: torch.zeros((), device=self.device)  # noqa: E731
      self._accum = dict(loss_sum=z(), z_sum=z(), weights=z(), aux=z(), micro=0)
      if compute_grads:
        store.begin_step()
    acc = self._accum
    acc["micro"] += 1
    for i in range(len(self._units)):          # a stage keeps its own units resident for the whole step
      self._gather(i, async_op=False)
    act_dtype = torch.bfloat16 if c.dtype == "bfloat16" else torch.float32
    sl = lambda t, m: None if t is None else t[m * mb:(m + 1) * mb]  # noqa: E731
    ctxs = [model.make_ctx(sl(positions, m), sl(seg, m), "train", sl(tokens, m)) for m in range(M)]
    aux_scale = None
    if self.n_moe_layers and c.load_balance_loss_weight > 0:
      # as in the base engine, and every micro-batch's balance loss is a mean over its own rows
      aux_scale = self._global_weight(weights.sum()) / self.n_moe_layers / self._data_shards() / M
    saved = {}          # (r, m) -> list of (layer, input, remat-saved tensors)
    final = {}          # m -> hidden state entering the head (last stage)
    # ---------------- forward
    for r in range(self.R):
      for m in range(M):
        if self._has_prev(r):
          x = self._recv((mb, S, c.emb_dim), act_dtype, self.prev_rank)
        else:
          x = self._run_embed(sl(tokens, m), sl(positions, m), grad=False)
        steps = []
        ctx = ctxs[m]
        for layer in self.chunks[r]:
          keep = {}
          ctx.saved, ctx.recompute, ctx.layer_index, ctx.aux_losses = keep, False, layer.index, []
          with torch.no_grad():
            y = layer(x, ctx)
          if ctx.aux_losses:
            acc["aux"] += sum(a for _, a in ctx.aux_losses).detach().float() / M
          steps.append((layer, x, keep))
          x = y
        saved[(r, m)] = steps
        if self._has_next(r):
          self._send(x, self.next_rank)
        else:
          final[m] = x
    self._drain()
    # ---------------- head + backward
    grads_started = not first
    for r in reversed(range(self.R)):
      for m in range(M):
        accumulate = grads_started or m > 0 or r < self.R - 1
        if self._has_next(r):
          dx = self._recv((mb, S, c.emb_dim), act_dtype, self.next_rank, "grad") if compute_grads else None
        else:
          hi = self._uidx["head"]
          if compute_grads:
            for u in self._units[hi]:
              store.acquire_full_grad(u)
          w = sl(weights, m).reshape(-1)
          loss_sum, z_sum, dx = self._run_head(final.pop(m), sl(targets, m).reshape(-1), w, compute_grads)
          acc["loss_sum"] += loss_sum
          acc["z_sum"] += z_sum
          acc["weights"] += w.sum()
          if compute_grads:
            self._finish_unit_grads(hi, accumulate and (m > 0 or grads_started), skip_embed=True)
        if not compute_grads:
          continue
        ctx = ctxs[m]
        for layer, x_in, keep in reversed(saved.pop((r, m))):
          ui = self._uidx[layer.unit]
          for u in self._units[ui]:
            store.acquire_full_grad(u)
          x_in = x_in.detach().requires_grad_(True)
          ctx.saved, ctx.recompute, ctx.layer_index, ctx.aux_losses = keep, True, layer.index, []
          with torch.enable_grad():
            y = layer(x_in, ctx)
            outs, gr = [y], [dx]
            if aux_scale is not None and ctx.aux_losses:
              for _, a in ctx.aux_losses:
                outs.append(a)
                gr.append(aux_scale.to(a.dtype))
          torch.autograd.backward(outs, gr)
          dx = x_in.grad
          for p in layer.params:
            p.collect_leaf_grad()
          self._finish_unit_grads(ui, grads_started or m > 0)
        if self._has_prev(r):
          self._send(dx, self.prev_rank, "grad")
        else:
          ei = self._uidx["embed"]
          for u in self._units[ei]:
            store.acquire_full_grad(u)
          self._run_embed(sl(tokens, m), sl(positions, m), grad=True, dx=dx)
          self._finish_unit_grads(ei, grads_started or m > 0)
    self._drain()
    if compute_grads:
      store.wait_reduce_scatters()
    for i in range(len(self._units)):          # the optimizer changes the shards: gather afresh next time
      self._release(i)
    return acc


def make_engine(config, mesh, device=None):
  """The engine that matches the mesh: pipelined when the `stage` axis is larger than one."""
  if mesh is not None and mesh.axis_size("stage") > 1:
    return PipelineEngine(config, mesh, device)
  return TrainEngine(config, mesh, device)
