"""Device mesh over one-process-per-GPU ranks.

MaxText builds a `jax.sharding.Mesh` of up to 12 named axes whose ICI degrees multiply to the
devices of a slice and whose DCN degrees multiply to the number of slices
(src/maxtext/utils/maxtext_utils.py:2154-2276, 2438). Here a mesh is a rank layout: the global rank
is the row-major index over `mesh_axes` (DCN-major, ICI-minor per axis), so the last axes
(`expert`, `tensor`, ...) are nearest neighbours, and every named axis (or tuple of axes) owns a
`torch.distributed` process group, NCCL on GPUs and gloo on CPU. Fused kernels additionally use
the symmetric-memory heap of `parallel.symm`.
"""
from __future__ import annotations

import datetime
import math
import os
from typing import Sequence

import torch
import torch.distributed as dist


def _env_int(*names, default=None):
  for n in names:
    v = os.environ.get(n)
    if v not in (None, ""):
      try:
        return int(v)
      except ValueError:
        continue
  return default


def init_distributed(timeout_s: int = 300, backend: str | None = None) -> tuple[int, int, int]:
  """Join the process group described by the environment; returns (rank, world, local_rank).

  Accepts torchrun variables (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT) and the
  variables of the reference's GPU launcher (JAX_COORDINATOR_IP / JAX_COORDINATOR_PORT / NNODES /
  NODE_RANK, tools/orchestration/gpu_multi_process_run.sh; src/maxtext/utils/max_utils.py:317-346).
  A single process without these variables stays un-initialised (world 1).
  """
  world = _env_int("WORLD_SIZE", "NNODES", default=1)
  rank = _env_int("RANK", "NODE_RANK", default=0)
  local_rank = _env_int("LOCAL_RANK", default=rank % max(1, torch.cuda.device_count() or 1))
  use_cuda = torch.cuda.is_available()
  if use_cuda:
    torch.cuda.set_device(local_rank % torch.cuda.device_count())
  if world <= 1:
    return 0, 1, local_rank
  if dist.is_initialized():
    return dist.get_rank(), dist.get_world_size(), local_rank
  if "MASTER_ADDR" not in os.environ:
    os.environ["MASTER_ADDR"] = os.environ.get("JAX_COORDINATOR_IP", "127.0.0.1")
  if "MASTER_PORT" not in os.environ:
    os.environ["MASTER_PORT"] = os.environ.get("JAX_COORDINATOR_PORT", "29511")
  backend = backend or ("nccl" if use_cuda else "gloo")
  kwargs = {}
  if backend == "nccl":
    kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
  dist.init_process_group(backend=backend, rank=rank, world_size=world,
                          timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
  return rank, world, local_rank


class Mesh:
  """Named-axis rank layout with lazily created process groups."""

  def __init__(self, axis_names: Sequence[str], shape: Sequence[int], rank: int | None = None, world: int | None = None):
    assert len(axis_names) == len(shape)
    self.axis_names = tuple(axis_names)
    self.shape = {a: int(n) for a, n in zip(axis_names, shape)}
    self.size = int(math.prod(shape))
    if world is None:
      world = dist.get_world_size() if dist.is_initialized() else 1
    if rank is None:
      rank = dist.get_rank() if dist.is_initialized() else 0
    if world != self.size:
      raise ValueError(f"mesh {dict(self.shape)} needs {self.size} ranks, process group has {world}")
    self.rank, self.world = rank, world
    self._groups: dict[tuple, object] = {}
    self._group_ranks: dict[tuple, list[int]] = {}

  # ---- coordinates
  def coords_of(self, rank: int) -> dict:
    out, rem = {}, rank
    for a in reversed(self.axis_names):
      out[a] = rem % self.shape[a]
      rem //= self.shape[a]
    return out

  def rank_of(self, coords: dict) -> int:
    r = 0
    for a in self.axis_names:
      r = r * self.shape[a] + coords.get(a, 0)
    return r

  @property
  def coords(self) -> dict:
    return self.coords_of(self.rank)

  def axis_size(self, axes) -> int:
    axes = (axes,) if isinstance(axes, str) else tuple(axes)
    return int(math.prod(self.shape.get(a, 1) for a in axes))

  def axis_index(self, axes) -> int:
    """Row-major index of this rank inside the sub-mesh spanned by `axes`."""
    axes = (axes,) if isinstance(axes, str) else tuple(axes)
    c, idx = self.coords, 0
    for a in axes:
      idx = idx * self.shape.get(a, 1) + c.get(a, 0)
    return idx

  def ranks_along(self, axes, rank: int | None = None) -> list[int]:
    """Global ranks that share all coordinates with `rank` except along `axes` (ordered by axis index)."""
    axes = (axes,) if isinstance(axes, str) else tuple(axes)
    axes = tuple(a for a in axes if a in self.shape)
    base = self.coords_of(self.rank if rank is None else rank)
    out = []
    sizes = [self.shape[a] for a in axes]
    for flat in range(int(math.prod(sizes)) if sizes else 1):
      c, rem = dict(base), flat
      for a, n in zip(reversed(axes), reversed(sizes)):
        c[a] = rem % n
        rem //= n
      out.append(self.rank_of(c))
    return out

  # ---- groups
  def group(self, axes):
    """Process group over `axes` containing this rank (None when the sub-mesh has one rank).

    Creation is collective: every rank must request the same axes in the same order.
    """
    axes = (axes,) if isinstance(axes, str) else tuple(axes)
    axes = tuple(a for a in self.axis_names if a in axes and self.shape[a] > 1)
    if not axes or self.world == 1:
      return None
    if axes in self._groups:
      return self._groups[axes]
    if len(axes) == sum(1 for a in self.axis_names if self.shape[a] > 1):
      self._groups[axes] = dist.group.WORLD
      self._group_ranks[axes] = list(range(self.world))
      return self._groups[axes]
    mine = None
    seen = set()
    for r in range(self.world):
      members = tuple(self.ranks_along(axes, r))
      if members in seen:
        continue
      seen.add(members)
      g = dist.new_group(list(members))
      if self.rank in members:
        mine = g
        self._group_ranks[axes] = list(members)
    self._groups[axes] = mine
    return mine

  def group_ranks(self, axes) -> list[int]:
    axes = (axes,) if isinstance(axes, str) else tuple(axes)
    return self.ranks_along(tuple(a for a in self.axis_names if a in axes and self.shape[a] > 1))

  def __repr__(self):
    nz = {a: n for a, n in self.shape.items() if n > 1}
    return f"Mesh({nz or '{}'}, rank={self.rank}/{self.world})"


def mesh_from_config(config, rank: int | None = None, world: int | None = None) -> Mesh:
  """Mesh whose per-axis size is ici x dcn degree (DCN-major ordering within each axis)."""
  return Mesh(list(config.mesh_axes), list(config.mesh_shape), rank=rank, world=world)
