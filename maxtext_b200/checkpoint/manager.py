"""Checkpoint save / restore in the reference's on-disk pytree layout.

Layout (src/maxtext/common/train_state_nnx.py:59-71, 140-178; src/maxtext/common/checkpointing.py:367-446,
944-1049): `<checkpoint_dir>/<step>/items/` holds the tree
`{"params": {"params": {...}}, "step": int32, "opt_state": [{count, mu: {params}, nu: {params}}]}` with
MaxText parameter names and shapes (`[in..., out...]` kernels; with `scan_layers` the layer axis is
stacked at `param_scan_axis`), `<step>/iter/` the data-iterator state, and a `commit_success.txt`
marker written last. Arrays are zarr v3 directories named by the '.'-joined tree path, one chunk per
layer so that every rank can write / read the layers it needs independently.

Restore priority (checkpointing.py:471-682): latest committed step in `checkpoint_dir` -> else
`load_parameters_path` (params only) -> else `load_full_state_path` -> else fresh init. Because arrays
are stored whole (not per-shard), a checkpoint restores onto any mesh: each rank reads the tensor and
keeps its own flat chunk.
"""
from __future__ import annotations

import concurrent.futures as cf
import json
import os
import shutil
import time

import numpy as np
import torch
import torch.distributed as dist

from ..parallel import param_store as ps
from ..utils import max_logging
from . import zarr3

COMMIT = "commit_success.txt"

try:
  import ml_dtypes
  _NP_BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
  _NP_BF16 = None


def _to_numpy(t: torch.Tensor) -> np.ndarray:
  t = t.detach().to("cpu")
  if t.dtype == torch.bfloat16:
    return t.view(torch.int16).numpy().view(_NP_BF16)
  return t.numpy()


def _from_numpy(a: np.ndarray) -> torch.Tensor:
  if _NP_BF16 is not None and a.dtype == _NP_BF16:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
  return torch.from_numpy(np.ascontiguousarray(a))


def leaf_key(pdef, scan_layers: bool, scan_axis: int = 1) -> tuple[tuple, int | None]:
  """Tree path of the array holding this parameter and the index of the layer axis (None if unstacked). With scanned layers
  the stacked layer axis sits at `param_scan_axis` of the array (src/maxtext/configs/base.yml `param_scan_axis`, default 1)."""
  if pdef.layer is None:
    return tuple(pdef.ref_path), None
  if scan_layers:
    return ("decoder", pdef.stack) + tuple(pdef.ref_path), int(scan_axis)
  return ("decoder", f"{pdef.stack}_{pdef.layer}") + tuple(pdef.ref_path), None


def _tp_slice_ref(pdef, mesh_tp_rank, mesh_tp_size, ep_rank, ep_size):
  """Slices of the (unstacked) reference tensor owned by this rank under tensor / expert parallelism."""
  sl = [slice(None)] * len(pdef.ref_shape)
  if pdef.kind == "linear" and pdef.tp_dim is not None and mesh_tp_size > 1:
    d = pdef.n_in_dims if pdef.tp_dim == 0 else 0   # internal dim 0 = out -> first out dim of ref
    n = pdef.ref_shape[d] // mesh_tp_size
    sl[d] = slice(mesh_tp_rank * n, (mesh_tp_rank + 1) * n)
  elif pdef.kind == "expert_linear":
    if pdef.ep_dim is not None and ep_size > 1:
      n = pdef.ref_shape[0] // ep_size
      sl[0] = slice(ep_rank * n, (ep_rank + 1) * n)
    if pdef.tp_dim is not None and mesh_tp_size > 1:
      d = 2 if pdef.tp_dim == 1 else 1
      n = pdef.ref_shape[d] // mesh_tp_size
      sl[d] = slice(mesh_tp_rank * n, (mesh_tp_rank + 1) * n)
  elif pdef.kind == "same" and pdef.tp_dim is not None and mesh_tp_size > 1:
    n = pdef.ref_shape[pdef.tp_dim] // mesh_tp_size
    sl[pdef.tp_dim] = slice(mesh_tp_rank * n, (mesh_tp_rank + 1) * n)
  return tuple(sl)


class TreeIO:
  """Maps store parameters <-> arrays of the reference tree on disk."""

  def __init__(self, engine, mesh):
    self.engine, self.mesh = engine, mesh
    self.store = engine.store
    self.c = engine.config
    self.rank = mesh.rank if mesh is not None else 0
    self.world = mesh.world if mesh is not None else 1
    par = engine.model.par
    self.tp_rank, self.tp_size, self.ep_rank, self.ep_size = par["tp_rank"], par["tp_size"], par["ep_rank"], par["ep_size"]

  def _local_ref_shape(self, pdef):
    sl = _tp_slice_ref(pdef, self.tp_rank, self.tp_size, self.ep_rank, self.ep_size)
    return tuple(len(range(*s.indices(n))) for s, n in zip(sl, pdef.ref_shape)), sl

  def _full_from_flat(self, p, flat):
    store = self.store
    u = store.unit_of(p)
    shard = store.shard_view(u, flat)
    if u.group_size > 1:
      full = torch.empty(u.numel, dtype=shard.dtype, device=shard.device)
      dist.all_gather_into_tensor(full, shard.contiguous(), group=u.group)
    else:
      full = shard
    off = u.offsets[u.params.index(p)]
    return full[off: off + p.pdef.numel].view(p.pdef.shape)

  def _array_dir(self, root, prefix, key):
    return os.path.join(root, ".".join(prefix + key))

  def write_tree(self, root: str, prefix: tuple, flat: torch.Tensor, pool, futures, dtype=None):
    """Write one store-aligned flat array (master weights, or a moment) as reference-layout zarr arrays."""
    scan = bool(self.c.scan_layers)
    stack_sizes = self.engine.model.stack_sizes
    written_meta = set()
    for i, p in enumerate(self.store.params.values()):
      d = p.pdef
      t = self._full_from_flat(p, flat)           # collective over the unit's shard group
      # one writer per distinct (tp, ep) slice: the first rank of each shard group
      u = self.store.unit_of(p)
      if not self._is_writer(p, u):
        continue
      ref_local = ps.to_ref_layout(_LocalView(d, self._local_ref_shape(d)[0]), t)
      arr = _to_numpy(ref_local.to(dtype) if dtype is not None else ref_local)
      key, axis = leaf_key(d, scan, int(self.c.param_scan_axis))
      adir = self._array_dir(root, prefix, key)
      shape = list(d.ref_shape)
      _, sl = self._local_ref_shape(d)
      if axis is not None:
        L = stack_sizes[d.stack]
        ax = min(axis, len(shape))
        shape.insert(ax, L)
        chunks = list(shape)
        chunks[ax] = 1
        # tp/ep slices become extra chunking of the split dims
        index = [0] * len(shape)
        index[ax] = d.layer
        ref_dims = [k for k in range(len(shape)) if k != ax]
        for rd, s, n in zip(ref_dims, sl, d.ref_shape):
          if s != slice(None):
            chunks[rd] = arr.shape[ref_dims.index(rd)]
            index[rd] = s.start // chunks[rd]
        block = np.expand_dims(arr, ax)
      else:
        chunks = list(shape)
        index = [0] * len(shape)
        for rd, (s, n) in enumerate(zip(sl, d.ref_shape)):
          if s != slice(None):
            chunks[rd] = arr.shape[rd]
            index[rd] = s.start // chunks[rd]
        block = arr
      if adir not in written_meta and self._is_meta_writer(d):
        zarr3.write_meta(adir, shape, chunks, arr.dtype)
        written_meta.add(adir)
      futures.append(pool.submit(zarr3.write_chunk, adir, tuple(index), block))

  def _is_writer(self, p, u) -> bool:
    """Exactly one rank writes each distinct chunk: the first rank of the unit's shard group, and among the ranks that hold
    identical copies (data-parallel replicas, tensor / expert ranks for parameters those axes do not split) the one at
    index 0 of every such axis. Pipeline stages hold different parameters, so every stage writes its own."""
    if u.group_rank != 0:
      return False
    m = self.mesh
    if m is None:
      return True
    d = p.pdef
    for a in m.axis_names:
      if m.shape[a] <= 1 or a in u.fsdp_axes or a == "stage":
        continue
      if a in ("tensor", "tensor_sequence") and d.tp_dim is not None:
        continue
      if a == "expert" and d.ep_dim is not None:
        continue
      if m.axis_index(a) != 0:
        return False
    return True

  def _is_meta_writer(self, d):
    first_layer = d.layer in (None, 0)
    return first_layer and self.tp_rank == 0 and self.ep_rank == 0 or (not self.c.scan_layers and self.tp_rank == 0 and self.ep_rank == 0)

  def _scan_axis_of(self, root: str) -> int:
    """The layer axis recorded by the writer of the tree under `root` (falls back to this run's `param_scan_axis`)."""
    cache = self.__dict__.setdefault("_scan_axis_cache", {})
    if root not in cache:
      ax = int(self.c.param_scan_axis)
      try:
        with open(os.path.join(root, "_METADATA"), "r", encoding="utf-8") as fh:
          ax = int(json.load(fh).get("custom_metadata", {}).get("param_scan_axis", ax))
      except (OSError, ValueError):
        pass
      cache[root] = ax
    return cache[root]

  def read_param(self, root: str, prefix: tuple, p) -> torch.Tensor | None:
    """Internal-layout tensor for parameter p from the tree under `root`, or None when absent."""
    d = p.pdef
    for scan in (bool(self.c.scan_layers), not bool(self.c.scan_layers)):
      key, axis = leaf_key(d, scan, self._scan_axis_of(root))
      adir = self._array_dir(root, prefix, key)
      if os.path.isfile(os.path.join(adir, "zarr.json")):
        break
    else:
      return None
    lshape, sl = self._local_ref_shape(d)
    region = list(sl)
    if axis is not None:
      ax = min(axis, len(d.ref_shape))
      region.insert(ax, slice(d.layer, d.layer + 1))
      arr = zarr3.read_array(adir, tuple(region))
      arr = np.squeeze(arr, ax)
    else:
      arr = zarr3.read_array(adir, tuple(region))
    t = _from_numpy(arr)
    return ps.from_ref_layout(_LocalView(d, lshape), t)


class _LocalView:
  """ParamDef look-alike whose ref_shape is the rank-local slice (for layout conversion under TP/EP)."""

  def __init__(self, d, local_ref_shape):
    self.kind, self.n_in_dims, self.shape, self.ref_shape = d.kind, d.n_in_dims, d.shape, tuple(local_ref_shape)


class CheckpointManager:
  def __init__(self, config, engine, mesh=None, directory: str | None = None):
    self.c, self.engine, self.mesh = config, engine, mesh
    self.dir = directory or config.checkpoint_dir
    self.rank = mesh.rank if mesh is not None else 0
    self.world = mesh.world if mesh is not None else 1
    self.io = TreeIO(engine, mesh)
    self.pool = cf.ThreadPoolExecutor(max_workers=8)
    self._inflight = None   # (step, futures, tmp_dir, final_dir)
    if self.rank == 0 and self.dir:
      os.makedirs(self.dir, exist_ok=True)
      self.cleanup_incomplete()

  # ------------------------------------------------------------------ discovery
  def all_steps(self, committed_only=True) -> list[int]:
    if not self.dir or not os.path.isdir(self.dir):
      return []
    out = []
    for n in os.listdir(self.dir):
      if n.isdigit() and (not committed_only or os.path.isfile(os.path.join(self.dir, n, COMMIT))):
        out.append(int(n))
    return sorted(out)

  def latest_step(self):
    s = self.all_steps()
    return s[-1] if s else None

  def cleanup_incomplete(self):
    """Remove step directories that lack the commit marker (a save that died half-way);
    src/maxtext/utils/elastic_utils.py:115-146 does the same before an elastic restart."""
    for n in os.listdir(self.dir):
      p = os.path.join(self.dir, n)
      if n.isdigit() and os.path.isdir(p) and not os.path.isfile(os.path.join(p, COMMIT)):
        shutil.rmtree(p, ignore_errors=True)

  # ------------------------------------------------------------------ save
  def should_save(self, step: int) -> bool:
    c = self.c
    if step == 0 and not c.save_checkpoint_on_start:
      return False
    return step % max(1, int(c.checkpoint_period)) == 0

  def maybe_save(self, step: int, data_iterator=None) -> bool:
    if self.should_save(step):
      self.save(step, data_iterator)
      return True
    return False

  def save_params_only(self, step: int = 0):
    """Parameters without optimizer state: what `load_parameters_path` consumers (decode, fine-tuning) need."""
    self.save(step, None, force=True, params_only=True)

  def save(self, step: int, data_iterator=None, force: bool = False, params_only: bool = False):
    if self._inflight is not None:
      self.wait_until_finished()
    if step in self.all_steps():
      return
    sdir = os.path.join(self.dir, str(step))
    items = os.path.join(sdir, "items")
    if self.rank == 0:
      os.makedirs(items, exist_ok=True)
    self._barrier()
    if self.engine.device.type == "cuda":
      torch.cuda.synchronize()
    futures = []
    store = self.engine.store
    self.io.write_tree(items, ("params", "params"), store.master, self.pool, futures)
    opt = {} if params_only else self.engine.optimizer.state_arrays()
    for name, flat in opt.items():
      self.io.write_tree(items, ("opt_state", "0", name, "params"), flat, self.pool, futures)
    if self.rank == 0:
      # the `step` leaf counts completed steps, as the reference's TrainState.step does after the step that is saved
      zarr3.write_array(os.path.join(items, "step"), np.asarray(step + 1, dtype=np.int32))
      zarr3.write_array(os.path.join(items, "opt_state.0.count"), np.asarray(self.engine.step_count, dtype=np.int32))
      meta = {"custom_metadata": {"scan_layers": bool(self.c.scan_layers), "param_scan_axis": int(self.c.param_scan_axis),
                                  "format": "zarr3", "use_ocdbt": False, "model_name": self.c.model_name},
              "tree_metadata": sorted(os.listdir(items)), "timestamp": time.time()}
      with open(os.path.join(items, "_METADATA"), "w", encoding="utf-8") as fh:
        json.dump(meta, fh)
    if data_iterator is not None and hasattr(data_iterator, "state"):
      # every rank records its own reader position: ranks of different data shards are at different places in the stream
      os.makedirs(os.path.join(sdir, "iter"), exist_ok=True)
      with open(os.path.join(sdir, "iter", f"process_{self.rank}.json"), "w", encoding="utf-8") as fh:
        json.dump(data_iterator.state(), fh)
    self._inflight = (step, futures, sdir)
    if not self.c.async_checkpointing or force:
      self.wait_until_finished()

  def wait_until_finished(self):
    if self._inflight is None:
      return
    step, futures, sdir = self._inflight
    for f in futures:
      f.result()
    self._barrier()
    if self.rank == 0:
      with open(os.path.join(sdir, COMMIT), "w", encoding="utf-8") as fh:
        fh.write(f"step {step} committed at {time.time()}\n")
      self._retain()
    self._inflight = None
    self._barrier()

  def _retain(self):
    keep = self.c.max_num_checkpoints_to_keep
    if keep is None:
      return
    steps = self.all_steps()
    for s in steps[:-int(keep)] if int(keep) > 0 else []:
      shutil.rmtree(os.path.join(self.dir, str(s)), ignore_errors=True)

  def _barrier(self):
    if self.world > 1 and dist.is_initialized():
      dist.barrier()

  # ------------------------------------------------------------------ restore
  def restore_if_possible(self, data_iterator=None):
    """Follows the restore priority chain; returns the step to resume from, or None for a fresh start."""
    c = self.c
    latest = self.latest_step()
    if latest is not None:
      self.restore(os.path.join(self.dir, str(latest)), full_state=True, data_iterator=data_iterator)
      max_logging.log(f"restored full state from step {latest}")
      return latest + 1
    if c.load_parameters_path:
      load_params_only(c.load_parameters_path, self.engine, self.mesh)
      return None
    if c.load_full_state_path:
      self.restore(c.load_full_state_path, full_state=True)
      return None
    return None

  def restore(self, step_dir: str, full_state: bool = True, data_iterator=None):
    items = os.path.join(step_dir, "items") if os.path.isdir(os.path.join(step_dir, "items")) else step_dir
    _restore_tree(self.io, items, self.engine, full_state)
    if data_iterator is not None and hasattr(data_iterator, "load_state"):
      it_file = os.path.join(step_dir, "iter", f"process_{self.rank}.json")
      if os.path.isfile(it_file):
        with open(it_file, "r", encoding="utf-8") as fh:
          data_iterator.load_state(json.load(fh))
      elif os.path.isfile(os.path.join(step_dir, "iter", "process_0.json")):
        # written by a run with fewer ranks: rank 0's position is the closest known one (exact only without packing windows)
        max_logging.log(f"warning: {step_dir} has no data-iterator state for rank {self.rank}; resuming from rank 0's position")
        with open(os.path.join(step_dir, "iter", "process_0.json"), "r", encoding="utf-8") as fh:
          data_iterator.load_state(json.load(fh))


def _restore_tree(io: TreeIO, items: str, engine, full_state: bool):
  store = engine.store
  missing = []
  for p in store.params.values():
    t = io.read_param(items, ("params", "params"), p)
    if t is None:
      missing.append(p.name)
      continue
    store.load_full(p.name, t.to(store.device))
  if not full_state:
    # a base-model checkpoint loaded under LoRA has no adapter tensors: those keep their initial value
    missing = [n for n in missing if not n.endswith(("_lora_a", "_lora_b"))]
  if missing:
    raise KeyError(f"checkpoint {items} lacks {len(missing)} parameters, e.g. {missing[:4]}")
  store.sync_compute_from_master()
  if full_state:
    opt = engine.optimizer.state_arrays()
    for name, flat in opt.items():
      for p in store.params.values():
        t = io.read_param(items, ("opt_state", "0", name, "params"), p)
        if t is None:
          continue
        u = store.unit_of(p)
        off = u.offsets[u.params.index(p)]
        lo, hi = u.group_rank * u.chunk, (u.group_rank + 1) * u.chunk
        a, b = max(off, lo), min(off + p.pdef.numel, hi)
        if a < b:
          store.shard_view(u, flat)[a - lo: b - lo].copy_(t.reshape(-1)[a - off: b - off].to(flat.dtype))
    cnt = os.path.join(items, "opt_state.0.count")
    if os.path.isdir(cnt):
      engine.step_count = int(zarr3.read_array(cnt))


def load_params_only(path: str, engine, mesh=None):
  """`load_parameters_path`: restore weights, keep a fresh optimizer (checkpointing.py:704-768)."""
  items = os.path.join(path, "items") if os.path.isdir(os.path.join(path, "items")) else path
  _restore_tree(TreeIO(engine, mesh), items, engine, full_state=False)


class MultiTierCheckpointManager:
  """Two tiers: frequent saves to node-local storage, rarer saves to the persistent directory; restore takes the newest
  committed step of either tier.

  The role of emergency / multi-tier checkpointing (src/maxtext/common/emergency_checkpointing.py; train_utils.py:54-114:
  `local_checkpoint_directory`, `local_checkpoint_period`, `enable_emergency_checkpoint`): after a restart on the same
  hosts the local copy saves a trip to shared storage; after losing hosts the persistent tier still has a recent step.
  Both tiers use the same on-disk tree, so either can feed `load_full_state_path`.
  """

  def __init__(self, config, engine, mesh=None):
    self.c = config
    self.persistent = CheckpointManager(config, engine, mesh)
    local_cfg = config.replace(checkpoint_period=max(1, int(config.local_checkpoint_period)),
                               max_num_checkpoints_to_keep=2 if config.max_num_checkpoints_to_keep is None else config.max_num_checkpoints_to_keep)
    self.local = CheckpointManager(local_cfg, engine, mesh, directory=config.local_checkpoint_directory)
    self.engine = engine

  def maybe_save(self, step, data_iterator=None) -> bool:
    a = self.persistent.maybe_save(step, data_iterator)
    b = False if a else self.local.maybe_save(step, data_iterator)      # a persistent save makes the local one redundant
    return a or b

  def save(self, step, data_iterator=None, force=False):
    self.persistent.save(step, data_iterator, force=force)

  def latest_step(self):
    steps = [s for s in (self.persistent.latest_step(), self.local.latest_step()) if s is not None]
    return max(steps) if steps else None

  def cleanup_incomplete(self):
    self.persistent.cleanup_incomplete()
    self.local.cleanup_incomplete()

  def wait_until_finished(self):
    self.persistent.wait_until_finished()
    self.local.wait_until_finished()

  def restore_if_possible(self, data_iterator=None):
    p, l = self.persistent.latest_step(), self.local.latest_step()
    if l is not None and (p is None or l > p):
      self.local.restore(os.path.join(self.local.dir, str(l)), full_state=True, data_iterator=data_iterator)
      max_logging.log(f"restored full state from local tier, step {l}")
      return l + 1
    return self.persistent.restore_if_possible(data_iterator)


def create_checkpoint_manager(config, engine, mesh=None):
  if config.enable_emergency_checkpoint and config.local_checkpoint_directory and int(config.local_checkpoint_period) > 0:
    return MultiTierCheckpointManager(config, engine, mesh)
  return CheckpointManager(config, engine, mesh)
