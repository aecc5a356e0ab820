"""Flat, unit-wise parameter storage with ZeRO-3 style sharding.

MaxText leaves parameter placement to GSPMD: each weight carries logical axis names, the rule table
maps them to mesh axes, and XLA inserts per-layer all-gathers / reduce-scatters
(src/maxtext/utils/sharding.py:362-469, docs/guides/optimization/sharding.md). Here placement is
explicit and laid out for NVLink collectives:

* every parameter belongs to a **unit** (embedding, one decoder layer, output head). All parameters
  of a unit live back to back in one flat buffer, so a layer's weights move with ONE all-gather and
  its gradients with ONE reduce-scatter, and adjacent tensors (q|k|v, wi_0|wi_1) can be consumed as
  one fused GEMM operand without a copy;
* the rule table still decides *which mesh axes* shard a parameter: tensor-like axes split a real
  dimension (handled by the layer code, the store sees the local shape), every other axis that the
  rules assign (fsdp, fsdp_transpose, context, expert-as-fsdp...) joins the unit's flat shard group:
  rank r of that group owns elements [r*chunk, (r+1)*chunk) of the flat unit;
* fp32 master weights, AdamW moments and fp32 gradient shards are single contiguous arrays over all
  units, so the optimizer is one kernel launch over the local shard;
* the compute-dtype copy of a unit is materialised into a small pool of gather buffers, prefetched
  one unit ahead by the step schedule of `train.engine.TrainEngine`.

Internal linear layout is `[out, in]`; the reference layout (`[in..., out...]`, layer axis stacked
at `param_scan_axis`) is produced by `to_reference_tree` for checkpoints.
"""
from __future__ import annotations

import os

import hashlib
import math
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch
import torch.distributed as dist

from . import rules as _rules

ALIGN = 256  # elements; keeps every parameter 512-byte aligned in bf16 (TMA needs 16 B)

_TP_AXES = ("tensor", "tensor_sequence", "autoregressive")
_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def torch_dtype(name) -> torch.dtype:
  return name if isinstance(name, torch.dtype) else _DTYPES[name]


@dataclass
class ParamDef:
  name: str                      # unique, e.g. "layers_3/self_attention/query/kernel"
  unit: str                      # "embed" | "layer_<i>" | "head" | ...
  shape: tuple                   # internal layout, local to this rank
  ref_path: tuple                # path in the reference tree (without layer index)
  ref_shape: tuple               # reference layout, global
  logical_axes: tuple            # logical names of the reference dims
  kind: str = "linear"           # "linear": ref [in..,out..] <-> internal [out,in]; "same": identical layout
  n_in_dims: int = 1             # for kind=linear: how many leading ref dims are "in"
  init: str = "fan_in_trunc"     # fan_in_trunc | fan_in_normal | embed | ones | zeros | const | normal | log_uniform_16
  init_scale: float = 1.0
  layer: int | None = None       # index along the stacked layer axis
  stack: str | None = None       # name of the stacked collection in the reference tree ("layers", "dense_layers"...)
  weight_decay: bool = True
  tp_partial: bool = False       # replicated over the tensor axes but fed rank-local data: its gradient is a partial sum
  frozen: bool = False           # never trained (base weights under LoRA): gradient forced to zero, no weight decay
  tp_dim: int | None = None      # internal dim split over tensor axes (already applied to `shape`)
  ep_dim: int | None = None      # internal dim split over the expert axis (already applied)
  fsdp_axes: tuple = ()          # mesh axes of the flat shard group (filled by the store)
  tp_rank: int = 0
  tp_size: int = 1
  ep_rank: int = 0
  ep_size: int = 1

  def global_shape(self) -> tuple:
    """Internal-layout shape before tensor / expert parallel slicing."""
    s = list(self.shape)
    if self.tp_dim is not None:
      s[self.tp_dim] *= self.tp_size
    if self.ep_dim is not None:
      s[self.ep_dim] *= self.ep_size
    return tuple(s)

  def local_slice(self, t):
    """This rank's tensor / expert parallel slice of a global internal-layout tensor."""
    if self.tp_dim is not None and self.tp_size > 1:
      n = self.shape[self.tp_dim]
      t = t.narrow(self.tp_dim, self.tp_rank * n, n)
    if self.ep_dim is not None and self.ep_size > 1:
      n = self.shape[self.ep_dim]
      t = t.narrow(self.ep_dim, self.ep_rank * n, n)
    return t

  @property
  def numel(self) -> int:
    return int(math.prod(self.shape))


class Param:
  """Handle given to layer code. `.data` is the compute-dtype tensor (valid while the unit is
  resident), `.main_grad` the fp32 gradient accumulator view (valid during backward)."""

  __slots__ = ("pdef", "_data", "main_grad", "grad_written", "_leaf", "unit", "lora")

  def __init__(self, pdef: ParamDef):
    self.pdef = pdef
    self._data: torch.Tensor | None = None
    self.main_grad: torch.Tensor | None = None
    self.grad_written = False
    self._leaf = None
    self.unit = None          # set by the store
    self.lora = None          # (A, B, scale) low-rank adapter params of a linear, see layers.blocks.Builder.linear

  @property
  def data(self):
    """The compute-dtype tensor. If the unit's all-gather was deferred so that it could be fused into the first
    GEMM that reads it, any other reader triggers the stand-alone gather here."""
    u = self.unit
    if u is not None and u.pending_ag:
      u.store.ensure_gathered(u)
    return self._data

  @data.setter
  def data(self, t):
    self._data = t

  def pending_unit(self):
    u = self.unit
    return u if (u is not None and u.pending_ag) else None

  @property
  def name(self):
    return self.pdef.name

  @property
  def frozen(self):
    return self.pdef.frozen

  @property
  def shape(self):
    return self.pdef.shape

  def leaf(self) -> torch.Tensor:
    """An autograd leaf aliasing `.data` for ops that rely on plain PyTorch differentiation; its
    `.grad` is folded into `main_grad` by `collect_leaf_grads` after the unit's backward."""
    if not torch.is_grad_enabled() or self.pdef.frozen:
      return self.data
    if self._leaf is None or self._leaf.data_ptr() != self.data.data_ptr():
      self._leaf = self.data.detach().requires_grad_(True)
    return self._leaf

  def accumulate_grad(self, g: torch.Tensor):
    if self.pdef.frozen:
      return
    if self.grad_written:
      self.main_grad.add_(g.reshape(self.main_grad.shape))
    else:
      self.main_grad.copy_(g.reshape(self.main_grad.shape))
      self.grad_written = True

  def collect_leaf_grad(self):
    if self._leaf is not None:
      if self._leaf.grad is not None:
        self.accumulate_grad(self._leaf.grad)
      self._leaf = None


@dataclass
class Unit:
  name: str
  fsdp_axes: tuple
  params: list = field(default_factory=list)     # list[Param]
  offsets: list = field(default_factory=list)
  numel: int = 0          # padded to a multiple of ALIGN * shard group size
  chunk: int = 0          # numel / shard group size
  shard_offset: int = 0   # offset of this unit's chunk in the local flat arrays
  group: object = None
  group_size: int = 1
  group_rank: int = 0
  full: torch.Tensor | None = None        # compute-dtype full buffer while resident
  full_grad: torch.Tensor | None = None   # fp32 full gradient buffer during backward
  resident: bool = False
  pending_ag: bool = False                # full buffer bound but not yet filled (fused all-gather mode)
  store: object = None
  grad_slot: int = -1                     # symmetric gradient buffer in use (fused reduce-scatter mode)


def _seed_for(name: str, base_seed: int) -> int:
  h = hashlib.sha256(f"{base_seed}:{name}".encode()).digest()
  return int.from_bytes(h[:7], "little")


def init_full_tensor(pdef: ParamDef, device, base_seed: int, mode: str = "reference", std: float = 0.02) -> torch.Tensor:
  """Deterministic fp32 initial value of the whole (local-TP) parameter, independent of FSDP degree.

  reference mode follows src/maxtext/layers/initializers.py:30-63 / linears.py:125 / attentions.py:276:
  variance_scaling(1.0, fan_in, truncated_normal | normal); `normal` mode draws N(0, std^2) for every
  matrix (the tiny-model and benchmark configurations)."""
  gen = torch.Generator(device="cpu" if str(device) == "cpu" else device)
  gen.manual_seed(_seed_for(pdef.name, base_seed))
  if pdef.init == "ones":
    return torch.ones(pdef.shape, dtype=torch.float32, device=device)
  if pdef.init == "zeros":
    return torch.zeros(pdef.shape, dtype=torch.float32, device=device)
  if pdef.init == "const":
    return torch.full(pdef.shape, float(pdef.init_scale), dtype=torch.float32, device=device)     # init_scale carries the constant
  if pdef.init == "log_uniform_16":
    # decay rates of the gated delta network: log of U(0, 16) (src/maxtext/models/qwen3.py:547-552)
    t = torch.empty(pdef.global_shape(), dtype=torch.float32, device=device).uniform_(1e-9, 16.0, generator=gen)
    return pdef.local_slice(torch.log(t)).contiguous()
  # draw the whole tensor, then keep this rank's tensor/expert-parallel slice: values do not depend on the mesh
  t = torch.empty(pdef.global_shape(), dtype=torch.float32, device=device)
  if mode == "normal" or pdef.init == "normal":
    t.normal_(0.0, std, generator=gen)
    return pdef.local_slice(t).contiguous() * pdef.init_scale
  if pdef.kind == "linear":
    fan_in = int(math.prod(pdef.ref_shape[:pdef.n_in_dims]))
  elif pdef.init == "embed":
    fan_in = pdef.ref_shape[-1]  # out_axis=0 -> fan_in is the feature dim
  else:
    fan_in = pdef.ref_shape[0]
  s = math.sqrt(1.0 / max(1, fan_in))
  if pdef.init == "fan_in_trunc":
    torch.nn.init.trunc_normal_(t, 0.0, 1.0, -2.0, 2.0, generator=gen)
    t.mul_(s / 0.87962566103423978)
  else:
    t.normal_(0.0, s, generator=gen)
  return pdef.local_slice(t).contiguous() * pdef.init_scale


class _EventWork:
  """`wait()` makes the current stream wait for a gather that ran on the gather stream (the engine's handle for prefetches)."""

  def __init__(self, event):
    self.event = event

  def wait(self):
    torch.cuda.current_stream().wait_event(self.event)


class ParamStore:
  def __init__(self, params: Sequence[Param], mesh, config, device, logical_rules=None):
    self.mesh, self.config, self.device = mesh, config, torch.device(device)
    self.compute_dtype = torch_dtype(config.dtype)
    self.weight_dtype = torch_dtype(config.weight_dtype)
    self.grad_dtype = torch_dtype(config.grad_dtype)
    self.mu_dtype = torch_dtype(config.mu_dtype)
    rules = logical_rules if logical_rules is not None else config.logical_axis_rules
    self.params: dict[str, Param] = {}
    self.units: dict[str, Unit] = {}
    self.specs: dict[str, _rules.ShardSpec] = {}
    mesh_shape = mesh.shape
    for p in params:
      d = p.pdef
      spec = _rules.make_spec(d.logical_axes, rules, mesh_shape, d.ref_shape)
      self.specs[d.name] = spec
      flat_axes = tuple(a for a in mesh.axis_names if a in spec.all_axes and a not in _TP_AXES and a != "stage"
                        and not (a == "expert" and d.ep_dim is not None))
      if config.shard_optimizer_over_data and mesh_shape.get("data", 1) > 1 and "data" not in flat_axes:
        flat_axes = tuple(a for a in mesh.axis_names if a in flat_axes or a == "data")
      d.fsdp_axes = flat_axes
      ukey = d.unit if not self.units.get(d.unit) or self.units[d.unit].fsdp_axes == flat_axes else f"{d.unit}#{'+'.join(flat_axes) or 'rep'}"
      if ukey not in self.units:
        self.units[ukey] = Unit(name=ukey, fsdp_axes=flat_axes)
      if d.name in self.params:
        raise ValueError(f"duplicate parameter name {d.name}")
      self.params[d.name] = p
      self.units[ukey].params.append(p)
      self.units[ukey].store = self
      p.unit = self.units[ukey]
    # layout
    total_local = 0
    for u in self.units.values():
      u.group_size = mesh.axis_size(u.fsdp_axes) if u.fsdp_axes else 1
      u.group_rank = mesh.axis_index(u.fsdp_axes) if u.fsdp_axes else 0
      off = 0
      for p in u.params:
        u.offsets.append(off)
        off += -(-p.pdef.numel // ALIGN) * ALIGN
      quantum = ALIGN * u.group_size
      u.numel = -(-off // quantum) * quantum
      u.chunk = u.numel // u.group_size
      u.shard_offset = total_local
      total_local += u.chunk
    self.local_numel = total_local
    dev = self.device
    self.master = torch.zeros(total_local, dtype=self.weight_dtype, device=dev)
    self.alias_compute = self.compute_dtype == self.weight_dtype
    # process groups (collective creation, deterministic order)
    for u in self.units.values():
      # planning runs build the store on the meta device for worlds that are not attached: no process groups there
      u.group = mesh.group(u.fsdp_axes) if (u.group_size > 1 and self.device.type != "meta") else None
    # ---- fused communication (symmetric memory over NVLink): when every sharded unit is sharded over the SAME group of ranks
    # (the whole world for pure FSDP; the ranks of one tensor / expert / pipeline coordinate on mixed meshes)
    self.fused = False
    self.symm = None
    world = getattr(mesh, "world", 1)
    sharded = [u for u in self.units.values() if u.group_size > 1]
    one_group = bool(sharded) and len({(tuple(u.fsdp_axes), u.group_size) for u in sharded}) == 1
    if (bool(getattr(config, "use_fused_comm_kernels", False)) and self.device.type == "cuda" and world > 1 and one_group
        and not self.alias_compute and self.compute_dtype == torch.bfloat16
        and self.grad_dtype == torch.float32 and not bool(config.logits_via_embedding)):
      from . import symm as _symm
      if _symm.available():
        try:
          whole = sharded[0].group_size == world
          self.symm = _symm.SymmGroup(None if whole else sharded[0].group, self.device)
          self.fused = True
        except Exception as e:  # pylint: disable=broad-except
          # no peer mapping on this platform (or the allocator refused): the NCCL composition below does the same job
          from ..utils import max_logging
          max_logging.log(f"symmetric memory unavailable ({e!r}); FSDP collectives use NCCL")
          self.symm, self.fused = None, False
    if self.fused:
      self._cs = self.symm.alloc(total_local, self.compute_dtype, zero=True)
      self.compute_shard = self._cs.tensor
      self.seg_elems = 512 * 1024
      max_chunk = max(u.chunk for u in sharded)
      gsz = sharded[0].group_size
      self.seg_flags = torch.zeros(gsz * (-(-max_chunk // self.seg_elems)), dtype=torch.int32, device=dev)
      # on a mixed mesh some tensors of a unit are replicated over the other axes: the gradient norm then weighs every tensor by
      # its multiplicity, which the partial sums emitted by the reduce-scatter kernels cannot do
      self.gradsq_whole_world = gsz == world
      self.comm_ctas = int(getattr(config, "fsdp_comm_ctas", 8))
      # How a unit's all-gather runs, one unit ahead of its first use and on its own stream in both default forms.
      # "dma": one peer-to-local copy per rank on the copy engines (no SM time); "prefetch": a peer-load kernel (32 CTAs).
      # "gemm": copier CTAs inside the first GEMM of the unit. "inline": the gather kernel on the compute stream at first use.
      # Measured on 8 GPUs (Llama-3-8B step): prefetch 1228 ms, dma 1156 ms; with in-switch reduction of the gradient
      # reduce-scatter 1188 and 1125 ms. On 2 GPUs: prefetch 1148 ms, dma 1140 ms, and plain peer loads beat the in-switch
      # reduction (1135 vs 1150 ms), which is therefore used from four ranks up.
      big = gsz >= 4
      self.ag_mode = os.environ.get("MAXTEXT_B200_AG_MODE", "dma")
      self.ag_in_gemm = self.ag_mode == "gemm"
      self.ag_stream = torch.cuda.Stream(device=dev)
      # in-switch (NVLS) reduction of the gradient reduce-scatter when the buffers have a multicast address: the switch adds the
      # copies (`multimem.ld_reduce`), so each rank receives one chunk instead of `world` of them
      self.rs_nvls = os.environ.get("MAXTEXT_B200_RS_NVLS", "1" if big else "0") == "1"
      self.comm_stream = torch.cuda.Stream(device=dev)
      self._gbufs = None
      self._gslot_pending = [None, None]
      self.gradsq = torch.zeros(1, dtype=torch.float32, device=dev)
      self.gradsq_valid = False
    else:
      self.compute_shard = self.master if self.alias_compute else torch.zeros(total_local, dtype=self.compute_dtype, device=dev)
    self.grad_shard = None   # allocated on first backward (inference never needs it)
    self.exp_avg = None
    self.exp_avg_sq = None
    self._pool: list[torch.Tensor] = []
    self._grad_pool: list[torch.Tensor] = []
    self._rs_inflight: list = []
    self.max_grad_buffers = 2
    self._bind_resident_units()

  # ------------------------------------------------------------------ views
  def _views_into(self, u: Unit, flat: torch.Tensor, attr: str):
    for p, off in zip(u.params, u.offsets):
      setattr(p, attr, flat[off: off + p.pdef.numel].view(p.pdef.shape))

  def _bind_resident_units(self):
    for u in self.units.values():
      if u.group_size == 1:
        u.full = self.compute_shard[u.shard_offset: u.shard_offset + u.numel]
        u.resident = True
        self._views_into(u, u.full, "data")

  def decay_slices(self):
    """None when weight decay applies to the whole shard; else the [a, b) ranges of this rank's flat shard that are decayed
    (trainable parameters that `adamw_mask` does not exclude)."""
    cached = getattr(self, "_decay", False)
    if cached is not False:
      return cached
    out = None
    if any(p.pdef.frozen or not p.pdef.weight_decay for u in self.units.values() for p in u.params):
      out = []
      for u in self.units.values():
        lo, hi = u.group_rank * u.chunk, (u.group_rank + 1) * u.chunk
        for p, off in zip(u.params, u.offsets):
          a, b = max(off, lo), min(off + p.pdef.numel, hi)
          if not p.pdef.frozen and p.pdef.weight_decay and a < b:
            out.append((u.shard_offset + a - lo, u.shard_offset + b - lo))
    self._decay = out
    return out

  def trainable_slices(self):
    """None when every parameter trains; else the [a, b) ranges of this rank's flat shard that belong to trainable ones."""
    cached = getattr(self, "_trainable", False)
    if cached is not False:
      return cached
    out = None
    if any(p.pdef.frozen for u in self.units.values() for p in u.params):
      out = []
      for u in self.units.values():
        lo, hi = u.group_rank * u.chunk, (u.group_rank + 1) * u.chunk
        for p, off in zip(u.params, u.offsets):
          a, b = max(off, lo), min(off + p.pdef.numel, hi)
          if not p.pdef.frozen and a < b:
            out.append((u.shard_offset + a - lo, u.shard_offset + b - lo))
    self._trainable = out
    return out

  def shard_view(self, u: Unit, flat: torch.Tensor) -> torch.Tensor:
    return flat[u.shard_offset: u.shard_offset + u.chunk]

  def ensure_grad_buffers(self):
    if self.grad_shard is None:
      self.grad_shard = torch.zeros(self.local_numel, dtype=self.grad_dtype, device=self.device)
      for u in self.units.values():
        if u.group_size == 1:
          u.full_grad = self.grad_shard[u.shard_offset: u.shard_offset + u.numel]
          self._views_into(u, u.full_grad, "main_grad")

  def ensure_opt_state(self):
    if self.exp_avg is None:
      self.exp_avg = torch.zeros(self.local_numel, dtype=self.mu_dtype, device=self.device)
      self.exp_avg_sq = torch.zeros(self.local_numel, dtype=torch.float32, device=self.device)

  # ------------------------------------------------------------------ init
  def initialize(self, seed: int = 0, mode: str | None = None, std: float | None = None):
    mode = mode or getattr(self.config, "weight_init", "reference")
    std = std if std is not None else getattr(self.config, "weight_init_std", 0.02)
    for u in self.units.values():
      lo, hi = u.group_rank * u.chunk, (u.group_rank + 1) * u.chunk
      dst = self.shard_view(u, self.master)
      for p, off in zip(u.params, u.offsets):
        n = p.pdef.numel
        a, b = max(off, lo), min(off + n, hi)
        if a >= b:
          continue
        full = init_full_tensor(p.pdef, self.device, seed, mode, std).reshape(-1)
        dst[a - lo: b - lo].copy_(full[a - off: b - off].to(self.weight_dtype))
        del full
    self.sync_compute_from_master()
    if self.fused:
      self.symm.barrier(0)        # every rank's shard is final before anyone reads it over NVLink

  def sync_compute_from_master(self):
    if not self.alias_compute:
      self.compute_shard.copy_(self.master)

  # ------------------------------------------------------------------ gather / scatter (synchronous forms; the
  # overlapped schedule is driven by train.engine.TrainEngine through prefetch / release)
  def max_unit_numel(self) -> int:
    return max((u.numel for u in self.units.values() if u.group_size > 1), default=0)

  def acquire_full(self, u: Unit) -> torch.Tensor:
    if self._pool:
      buf = self._pool.pop()
    else:
      buf = torch.empty(self.max_unit_numel(), dtype=self.compute_dtype, device=self.device)
    return buf[: u.numel]

  def release_full(self, u: Unit):
    if u.group_size > 1 and u.full is not None:
      self._pool.append(u.full._base if u.full._base is not None else u.full)
      u.full, u.resident, u.pending_ag = None, False, False
      for p in u.params:
        p.data = None

  def gather_unit(self, u: Unit, async_op: bool = False):
    """All-gather the compute-dtype shards of unit `u` into a pooled full buffer."""
    if u.group_size == 1 or u.resident:
      return None
    if self.fused:
      buf = self.acquire_full(u)
      u.full, u.resident = buf, True
      self._views_into(u, buf, "data")
      if self.ag_mode in ("prefetch", "dma"):
        # gather now, on the gather stream: it may start as soon as the compute stream no longer reads this pooled buffer
        from ..ops import backend
        # order after everything already enqueued on the compute stream: the previous user of this pooled buffer and, at the
        # start of a step, the optimizer update of the shards. The engine issues the prefetch BEFORE it enqueues the current
        # unit's kernels, so the copy still overlaps that unit's compute.
        self.ag_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.ag_stream):
          esz = u.full.element_size()
          if self.ag_mode == "dma":
            # copy engines instead of SMs: one peer-to-local copy per rank, the compute kernels keep every SM
            ptrs = [int(a) + u.shard_offset * esz for a in self._cs.ptrs]
            backend.ext().gather_dma(ptrs, u.full, u.chunk * esz, (self.symm.rank + 1) % u.group_size)
          else:
            backend.ext().gather_segments(self.peer_table(u), u.full, u.chunk * esz, self.seg_elems * esz, u.group_size, 32)
          done = torch.cuda.Event()
          done.record(self.ag_stream)
        if not async_op:
          torch.cuda.current_stream().wait_event(done)
          return None
        return _EventWork(done)
      # defer: the first GEMM that reads the unit gathers it inside its own launch (see ag_linear)
      u.pending_ag = True
      return None
    buf = self.acquire_full(u)
    work = dist.all_gather_into_tensor(buf, self.shard_view(u, self.compute_shard), group=u.group, async_op=async_op)
    u.full = buf
    u.resident = True
    self._views_into(u, buf, "data")
    return work

  # ------------------------------------------------------------------ fused paths (symmetric memory)
  def peer_table(self, u: Unit) -> torch.Tensor:
    """Device table with every rank's address of this unit's compute-dtype shard."""
    t = getattr(u, "_peer_table", None)
    if t is None:
      t = self._cs.table_at(u.shard_offset)
      u._peer_table = t
    return t

  def ensure_gathered(self, u: Unit):
    """Stand-alone all-gather by peer loads (used when the first reader of a unit is not a GEMM)."""
    if not u.pending_ag:
      return
    u.pending_ag = False
    from ..ops import backend
    esz = u.full.element_size()
    backend.ext().gather_segments(self.peer_table(u), u.full, u.chunk * esz, self.seg_elems * esz, u.group_size, 64)

  def ag_linear(self, u: Unit, p, x2: torch.Tensor):
    """y = x2 @ W.T where W is a parameter (or a run of adjacent parameters) of a unit whose all-gather is still
    pending: one launch copies the peers' shards of the whole unit and computes the product, tile by tile as rows
    arrive. Returns None when the shapes do not fit the fused kernel (the caller then gathers and multiplies)."""
    first = p.parts[0] if hasattr(p, "parts") else p
    N, K = p.shape
    M = x2.shape[0]
    if not self.ag_in_gemm:
      return None
    if not (x2.is_cuda and x2.dtype == torch.bfloat16 and M >= 128 and N >= 256 and K >= 64 and K % 8 == 0 and x2.stride(1) == 1):
      return None
    from ..ops import backend
    off = u.offsets[u.params.index(first)]
    out = torch.empty(M, N, dtype=x2.dtype, device=x2.device)
    u.pending_ag = False
    backend.ext().gemm_ag(x2, out, self.peer_table(u), u.full, N, K, u.chunk, self.seg_elems, off, u.group_size, self.seg_flags,
                          self.comm_ctas)
    return out

  def _fused_acquire_grad(self, u: Unit):
    if self._gbufs is None:
      n = self.max_unit_numel()
      self._gbufs = [self.symm.alloc(n, self.grad_dtype), self.symm.alloc(n, self.grad_dtype)]
      self._next_slot = 0
    b = self._next_slot
    self._next_slot ^= 1
    pend = self._gslot_pending[b]
    if pend is not None:
      ev, epoch = pend
      torch.cuda.current_stream().wait_event(ev)          # my own reduction of this buffer has finished
      self.symm.wait(3 + 2 * b, epoch)                    # and every peer has finished reading my copy
      self._gslot_pending[b] = None
    u.grad_slot = b
    u.full_grad = self._gbufs[b].tensor[: u.numel]
    self._views_into(u, u.full_grad, "main_grad")
    self._zero_gaps(u)
    for p in u.params:
      p.grad_written = False

  def _fused_reduce_scatter(self, u: Unit, accumulate: bool):
    from ..ops import backend
    for p in u.params:
      if not p.grad_written or p.pdef.frozen:
        p.main_grad.zero_()
    b = u.grad_slot
    dst = self.shard_view(u, self.grad_shard)
    main = torch.cuda.current_stream()
    ready = torch.cuda.Event()
    ready.record(main)
    with torch.cuda.stream(self.comm_stream):
      self.comm_stream.wait_event(ready)
      self.symm.signal(2 + 2 * b)                         # my gradients for this buffer are complete
      self.symm.wait(2 + 2 * b)                           # ... and so are everyone else's
      gb = self._gbufs[b]
      if self.rs_nvls and gb.mc_ptr:
        # one multimem.ld_reduce per element: the NVSwitch adds the ranks' copies, this GPU reads only its own chunk
        backend.ext().rs_sumsq_mc(gb.mc_ptr, u.group_rank * u.chunk, u.chunk, dst, bool(accumulate), 1.0,
                                  self.gradsq if self.gradsq_valid else None, 32)
      else:
        backend.ext().rs_sumsq(gb.table, u.group_rank * u.chunk, u.chunk, dst, bool(accumulate), 1.0, u.group_size,
                               self.gradsq if self.gradsq_valid else None, 48)
      epoch = self.symm.signal(3 + 2 * b)                 # I am done reading the peers' copies
      done = torch.cuda.Event()
      done.record(self.comm_stream)
    self._gslot_pending[b] = (done, epoch)
    self._rs_inflight.append((None, None, None, done))
    u.full_grad, u.grad_slot = None, -1
    for p in u.params:
      p.main_grad = None

  def acquire_full_grad(self, u: Unit):
    """Bind a full-size gradient buffer to unit `u`. At most two buffers exist: when both are busy the
    oldest in-flight reduce-scatter is completed first."""
    if u.group_size == 1:
      return
    if self.fused:
      return self._fused_acquire_grad(u)
    if not self._grad_pool and len(self._rs_inflight) >= self.max_grad_buffers - 1 and self._rs_inflight:
      self._complete_oldest_rs()
    if self._grad_pool:
      buf = self._grad_pool.pop()
    else:
      buf = torch.empty(self.max_unit_numel(), dtype=self.grad_dtype, device=self.device)
    u.full_grad = buf[: u.numel]
    self._views_into(u, u.full_grad, "main_grad")
    self._zero_gaps(u)
    for p in u.params:
      p.grad_written = False

  def _zero_gaps(self, u: Unit):
    """Alignment padding between parameters is reduced and normed with everything else: it must hold zeros."""
    gaps = getattr(u, "_gaps", None)
    if gaps is None:
      gaps, ends = [], [o + p.pdef.numel for o, p in zip(u.offsets, u.params)]
      for end, nxt in zip(ends, list(u.offsets[1:]) + [u.numel]):
        if nxt > end:
          gaps.append((end, nxt))
      u._gaps = gaps
    for lo, hi in gaps:
      u.full_grad[lo:hi].zero_()

  def reduce_scatter_unit(self, u: Unit, async_op: bool = True, accumulate: bool = False):
    """Sum the unit's full gradient over the shard group into this rank's gradient shard.

    The collective is launched asynchronously (it overlaps the backward of the next unit); the full
    buffer returns to the pool when the work item is completed by `acquire_full_grad` or
    `wait_reduce_scatters`."""
    if u.group_size == 1:
      return
    if self.fused:
      return self._fused_reduce_scatter(u, accumulate)
    for p in u.params:              # parameters never touched this step, and frozen ones, contribute zeros
      if not p.grad_written or p.pdef.frozen:
        p.main_grad.zero_()
    dst = self.shard_view(u, self.grad_shard)
    full = u.full_grad
    if accumulate:
      tmp = torch.empty_like(dst)
      work = dist.reduce_scatter_tensor(tmp, full, group=u.group, async_op=async_op)
      self._rs_inflight.append((work, full, dst, tmp))
    else:
      work = dist.reduce_scatter_tensor(dst, full, group=u.group, async_op=async_op)
      self._rs_inflight.append((work, full, None, None))
    u.full_grad = None
    for p in u.params:
      p.main_grad = None
    if not async_op:
      self.wait_reduce_scatters()

  def _complete_oldest_rs(self):
    work, full, dst, tmp = self._rs_inflight.pop(0)
    if full is None:                # fused path: `tmp` is the completion event of the reduction on the comm stream
      torch.cuda.current_stream().wait_event(tmp)
      return
    if work is not None:
      work.wait()
    if tmp is not None:
      dst.add_(tmp)
    self._grad_pool.append(full._base if full._base is not None else full)

  def wait_reduce_scatters(self):
    while self._rs_inflight:
      self._complete_oldest_rs()

  def release_full_grad(self, u: Unit):
    if u.group_size > 1 and u.full_grad is not None:
      self._grad_pool.append(u.full_grad._base if u.full_grad._base is not None else u.full_grad)
      u.full_grad = None
      for p in u.params:
        p.main_grad = None

  def begin_step(self):
    """Reset per-step gradient bookkeeping (resident units overwrite on first write)."""
    self.ensure_grad_buffers()
    if self.fused:
      self.gradsq.zero_()
      self.gradsq_valid = int(self.config.gradient_accumulation_steps) == 1 and self.gradsq_whole_world
    for u in self.units.values():
      for p in u.params:
        p.grad_written = False

  def finish_resident_grads(self):
    for u in self.units.values():
      if u.group_size == 1:
        for p in u.params:
          if not p.grad_written or p.pdef.frozen:
            p.main_grad.zero_()
            p.grad_written = True

  # ------------------------------------------------------------------ replica (data-parallel) reduction
  def replica_axes(self, u: Unit, params=None) -> tuple:
    """Mesh axes over which this unit's parameters (or the given ones of it) are replicated while the batch is split."""
    batch_axes = ("data", "fsdp", "fsdp_transpose", "expert", "context", "context_usp_ulysses", "stage")
    used = set(u.fsdp_axes)
    for p in (u.params if params is None else params):
      used.update(self.specs[p.name].all_axes)
    return tuple(a for a in self.mesh.axis_names if a in batch_axes and self.mesh.shape[a] > 1 and a not in used
                 and a != "stage")

  # ------------------------------------------------------------------ full tensors / reference tree
  def full_master(self, p: Param) -> torch.Tensor:
    """fp32 master value of one whole parameter (collective over the unit's shard group)."""
    u = self.unit_of(p)
    shard = self.shard_view(u, self.master)
    if u.group_size > 1:
      full = torch.empty(u.numel, dtype=shard.dtype, device=shard.device)
      dist.all_gather_into_tensor(full, shard.contiguous(), group=u.group)
    else:
      full = shard
    off = u.offsets[u.params.index(p)]
    return full[off: off + p.pdef.numel].view(p.pdef.shape)

  def unit_of(self, p: Param) -> Unit:
    for u in self.units.values():
      if p in u.params:
        return u
    raise KeyError(p.name)

  def load_full(self, name: str, value: torch.Tensor):
    """Set a parameter from a whole internal-layout tensor; every rank keeps its own chunk."""
    p = self.params[name]
    u = self.unit_of(p)
    off = u.offsets[u.params.index(p)]
    lo, hi = u.group_rank * u.chunk, (u.group_rank + 1) * u.chunk
    a, b = max(off, lo), min(off + p.pdef.numel, hi)
    if a < b:
      flat = value.reshape(-1)
      self.shard_view(u, self.master)[a - lo: b - lo].copy_(flat[a - off: b - off].to(self.weight_dtype))

  def named_specs(self) -> dict:
    return dict(self.specs)

  def num_parameters(self) -> int:
    return sum(p.pdef.numel for p in self.params.values())


# ---------------------------------------------------------------------- reference layout conversion
def to_ref_layout(pdef: ParamDef, t: torch.Tensor) -> torch.Tensor:
  if pdef.kind == "linear":
    n_in = int(math.prod(pdef.ref_shape[:pdef.n_in_dims]))
    return t.reshape(-1, n_in).t().reshape(pdef.ref_shape)
  if pdef.kind == "expert_linear":   # internal [E, out, in] <-> ref [E, in, out]
    return t.transpose(-1, -2).reshape(pdef.ref_shape)
  return t.reshape(pdef.ref_shape)


def from_ref_layout(pdef: ParamDef, t: torch.Tensor) -> torch.Tensor:
  if pdef.kind == "linear":
    n_in = int(math.prod(pdef.ref_shape[:pdef.n_in_dims]))
    return t.reshape(n_in, -1).t().contiguous().reshape(pdef.shape)
  if pdef.kind == "expert_linear":
    return t.reshape(pdef.ref_shape).transpose(-1, -2).contiguous().reshape(pdef.shape)
  return t.reshape(pdef.shape)
