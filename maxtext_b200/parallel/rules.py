"""Logical-axis -> mesh-axis resolution and per-tensor shard specifications.

Semantics follow what MaxText obtains from Flax (`nn.logical_to_mesh_axes`, used at
src/maxtext/utils/sharding.py:362-365) plus its own post-processing:

* the rule list is scanned **in rule order**; a rule ``(name, mesh_axes)`` is applied to the first
  dimension carrying that logical name if that dimension is still unassigned and none of the rule's
  mesh axes has been taken by another dimension of the same tensor. This is why the default table
  repeats names with smaller and smaller axis tuples: later entries are fallbacks;
* a dimension without an applicable rule is replicated;
* mesh axes of size one are dropped afterwards (sharding.py:182 `remove_size_one_mesh_axis`);
* a dimension whose extent is not divisible by the product of its mesh axes is replicated
  (sharding.py:237 `adjust_pspec_for_indivisible_shapes`).

The result is a :class:`ShardSpec`: for every tensor dimension the tuple of mesh axes it is split
over (major to minor). The planner and the FSDP / TP / EP engines consume these specs; nothing here
touches a device.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterable, Sequence


def _as_tuple(v) -> tuple:
  if v is None:
    return ()
  if isinstance(v, str):
    return (v,)
  return tuple(v)


def normalize_rules(rules: Iterable) -> list[tuple[str, tuple]]:
  return [(str(name), _as_tuple(axes)) for name, axes in rules]


def logical_to_mesh_axes(logical_names: Sequence[str | None], rules: Iterable) -> list[tuple]:
  """Resolve each dimension's logical name to a tuple of mesh axes (possibly empty)."""
  names = list(logical_names)
  unassigned = object()
  result: list = [unassigned] * len(names)
  for i, n in enumerate(names):
    if n is None:
      result[i] = ()
  used: set[str] = set()
  for rule_name, rule_axes in normalize_rules(rules):
    if rule_name not in names:
      continue
    pos = names.index(rule_name)
    if result[pos] is not unassigned:
      continue
    if any(a in used for a in rule_axes):
      continue
    result[pos] = rule_axes
    used.update(rule_axes)
  return [() if r is unassigned else r for r in result]


@dataclass(frozen=True)
class ShardSpec:
  """Per-dimension mesh axes of one tensor, after size-one and divisibility clean-up."""
  dims: tuple  # tuple[tuple[str, ...], ...]
  shape: tuple | None = None

  def axes_of(self, dim: int) -> tuple:
    return self.dims[dim]

  @property
  def all_axes(self) -> tuple:
    return tuple(a for d in self.dims for a in d)

  def degree(self, dim: int, mesh_shape: dict) -> int:
    return int(math.prod(mesh_shape[a] for a in self.dims[dim]))

  def total_degree(self, mesh_shape: dict) -> int:
    return int(math.prod(mesh_shape[a] for a in self.all_axes))

  def local_shape(self, mesh_shape: dict) -> tuple:
    assert self.shape is not None
    return tuple(s // self.degree(i, mesh_shape) for i, s in enumerate(self.shape))

  def dim_sharded_by(self, axis: str) -> int | None:
    for i, d in enumerate(self.dims):
      if axis in d:
        return i
    return None

  def to_json(self):
    return [list(d) if d else None for d in self.dims]


def make_spec(logical_names: Sequence[str | None], rules: Iterable, mesh_shape: dict,
              shape: Sequence[int] | None = None) -> ShardSpec:
  raw = logical_to_mesh_axes(logical_names, rules)
  dims = []
  for i, axes in enumerate(raw):
    axes = tuple(a for a in axes if mesh_shape.get(a, 1) > 1)
    if shape is not None and axes:
      deg = int(math.prod(mesh_shape[a] for a in axes))
      if shape[i] % deg:
        axes = ()
    dims.append(axes)
  return ShardSpec(tuple(dims), tuple(shape) if shape is not None else None)


# axes over which parameters are expected to be split when the axis is non-trivial
# (src/maxtext/utils/sharding.py:458-469)
_PARAM_SHARD_AXES = ("fsdp", "fsdp_transpose", "context", "tensor", "tensor_sequence", "stage", "expert", "sequence")


def unsharded_fraction(named_specs: dict, mesh_shape: dict) -> float:
  """Fraction of parameter elements that are not split over every non-trivial parameter axis."""
  active = [a for a in _PARAM_SHARD_AXES if mesh_shape.get(a, 1) > 1]
  if not active:
    return 0.0
  full = int(math.prod(mesh_shape[a] for a in active))
  total = 0
  per_device = 0
  for spec in named_specs.values():
    n = int(math.prod(spec.shape))
    total += n
    per_device += n // max(1, spec.total_degree(mesh_shape))
  perfect = total / full
  return (per_device - perfect) / max(1.0, total)


def assert_params_sufficiently_sharded(named_specs: dict, mesh_shape: dict, tolerance: float) -> None:
  """Fail when more than `tolerance` of the parameter volume sits replicated on each device
  (src/maxtext/utils/sharding.py:591)."""
  frac = unsharded_fraction(named_specs, mesh_shape)
  if frac > tolerance:
    raise AssertionError(
        f"Unsharded parameter fraction {frac:.4f} exceeds sharding_tolerance {tolerance}; "
        "check logical_axis_rules / parallelism degrees")
