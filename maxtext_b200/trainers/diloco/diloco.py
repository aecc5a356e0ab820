"""DiLoCo: replicas train independently for H inner steps, then agree through an outer Nesterov-SGD step.

Counterpart of src/maxtext/trainers/diloco/diloco.py:48-299 (vanilla and streaming train steps) and
trainers/diloco/utils/spmd_diloco_sync.py:31-124. There the inner state carries a leading replica dimension and the
inner step is vmapped over it; here each replica is a set of ranks (all mesh axes except `diloco`) that runs the
ordinary engine, gradients are never reduced across `diloco`, and the only cross-replica traffic is one all-reduce
of the parameter delta (`outer - inner`) over the `diloco` process group every `diloco_sync_period` steps -- on the
flat fp32 master shard, so ZeRO-3 sharding divides the volume by the shard count.

Streaming form (enable_streaming_diloco): the parameters are cut into `num_diloco_fragments` fragments (fragment 0:
embedding/head, the others: layers strided or sequential, fragmenter.py:72-81); one fragment is synchronised every
sync_period / num_fragments steps, its all-reduce runs on a side stream while `num_communication_overlapping_steps`
inner steps continue, and the result is mixed into the inner parameters as alpha * inner + (1 - alpha) * outer.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def nesterov_outer_step(outer: torch.Tensor, trace: torch.Tensor, pseudo_grad: torch.Tensor, lr: float, momentum: float):
  """optax.sgd(lr, momentum, nesterov=True) in place: trace = g + mu * trace; outer -= lr * (g + mu * trace)."""
  trace.mul_(momentum).add_(pseudo_grad)
  outer.add_(pseudo_grad + momentum * trace, alpha=-lr)


def streaming_schedule(config) -> tuple[int, int]:
  """(steps between fragment syncs, period) as in fragmenter.py:267-273."""
  nf = int(config.num_diloco_fragments)
  between = max(1, int(round(config.diloco_sync_period / nf)))
  return between, nf * between


def fragments_of(engine, config) -> list[list]:
  """Store units per fragment. Fragment 0 holds everything outside the layer stack."""
  nf = int(config.num_diloco_fragments or 0)
  n_layers = len(engine.model.layers)
  if nf < 2:
    raise ValueError("num_diloco_fragments must be at least 2 (one for embedding/head, at least one for the layers)")
  if n_layers % (nf - 1):
    raise ValueError(f"layers ({n_layers}) must divide by num_diloco_fragments - 1 ({nf - 1})")
  per = n_layers // (nf - 1)
  frag_of_layer = {}
  for f in range(1, nf):
    idx = range((f - 1) * per, f * per) if config.use_sequential_layers else range(f - 1, n_layers, nf - 1)
    for i in idx:
      frag_of_layer[i] = f
  out = [[] for _ in range(nf)]
  for name, u in engine.store.units.items():
    base = name.split("#")[0]
    f = frag_of_layer[int(base.split("_")[1])] if base.startswith("layer_") else 0
    out[f].append(u)
  return out


class DiLoCoTrainer:
  """Wraps a TrainEngine whose mesh has a `diloco` axis (or `replica_mean` for in-process replicas in tests)."""

  def __init__(self, engine, config, mesh=None, replica_mean=None):
    self.engine, self.c, self.mesh = engine, config, mesh
    st = engine.store
    self.group = mesh.group("diloco") if (mesh is not None and mesh.axis_size("diloco") > 1) else None
    self.replicas = mesh.axis_size("diloco") if mesh is not None else 1
    self._mean = replica_mean
    self.outer = st.master.detach().clone().float()
    self.trace = torch.zeros_like(self.outer)
    self.streaming = bool(config.enable_streaming_diloco)
    if self.streaming:
      self.frags = fragments_of(engine, config)
      self.between, self.period = streaming_schedule(config)
      self.delay = int(config.num_communication_overlapping_steps)
      self.alpha = float(config.communication_overlapping_alpha)
      self._inflight = {}
    self.side = torch.cuda.Stream() if st.master.is_cuda else None

  # ---- pieces
  def _ranges(self, units):
    return [(u.shard_offset, u.shard_offset + u.chunk) for u in units]

  def _reduce_mean(self, t: torch.Tensor, async_op: bool = False):
    if self._mean is not None:
      t.copy_(self._mean(t))
      return None
    if self.group is None:
      return None
    w = dist.all_reduce(t, group=self.group, async_op=async_op)
    t.div_(self.replicas) if not async_op else None
    return w

  def _outer_update(self, lo, hi, pseudo):
    nesterov_outer_step(self.outer[lo:hi], self.trace[lo:hi], pseudo, float(self.c.diloco_outer_lr), float(self.c.diloco_outer_momentum))

  def synchronize_full_state(self):
    st = self.engine.store
    pseudo = self.outer - st.master.float()
    self._reduce_mean(pseudo)
    self._outer_update(0, pseudo.numel(), pseudo)
    st.master.copy_(self.outer)
    st.sync_compute_from_master()

  def _sync_fragment(self, f: int):
    st = self.engine.store
    parts = []
    for lo, hi in self._ranges(self.frags[f]):
      parts.append(self.outer[lo:hi] - st.master[lo:hi].float())
    flat = torch.cat(parts) if parts else torch.zeros(0, device=self.outer.device)
    work = None
    if self.side is not None and self.group is not None:
      self.side.wait_stream(torch.cuda.current_stream())
      with torch.cuda.stream(self.side):                # the all-reduce overlaps the following inner steps
        work = dist.all_reduce(flat, group=self.group, async_op=True)
    else:
      self._reduce_mean(flat)
    self._inflight[f] = (flat, work, work is not None)

  def _finish_fragment(self, f: int):
    flat, work, scale = self._inflight.pop(f)
    if work is not None:
      work.wait()
    if scale:
      flat.div_(self.replicas)
    o = 0
    for lo, hi in self._ranges(self.frags[f]):
      self._outer_update(lo, hi, flat[o:o + hi - lo])
      o += hi - lo

  def _apply_fragment(self, f: int):
    if f in self._inflight:
      self._finish_fragment(f)
    st = self.engine.store
    for lo, hi in self._ranges(self.frags[f]):
      if self.alpha > 0:
        st.master[lo:hi].mul_(self.alpha).add_(self.outer[lo:hi].to(st.master.dtype), alpha=1 - self.alpha)
      else:
        st.master[lo:hi].copy_(self.outer[lo:hi])
    st.sync_compute_from_master()

  # ---- the step
  def train_step(self, batch) -> dict:
    metrics = self.engine.train_step(batch)
    step = self.engine.step_count
    if not self.streaming:
      if step % int(self.c.diloco_sync_period) == 0:
        self.synchronize_full_state()
      return metrics
    if step > 0 and step % self.between == 0:
      f = (step % self.period) // self.between
      self._sync_fragment(f)
      if self.delay == 0:
        self._finish_fragment(f)
    s = step - self.delay
    if s > 0 and s % self.between == 0:
      self._apply_fragment((s % self.period) // self.between)
    return metrics

  def state_arrays(self) -> dict:
    return {"outer_params": self.outer, "outer_trace": self.trace}
