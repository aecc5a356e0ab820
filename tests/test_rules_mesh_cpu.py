"""Logical-axis resolution, shard specs, mesh coordinates, and a golden sharding dump for the benchmark models."""
import json
import os

import pytest

from helpers import BASE_YML, ROOT
from maxtext_b200.config import pyconfig
from maxtext_b200.parallel import rules as R
from maxtext_b200.parallel.mesh import Mesh


def cfg(*a, n=8):
  return pyconfig.initialize(["t", BASE_YML, "log_config=false", *a], num_devices=n)


def test_rule_order_decides_and_axes_are_used_once():
  c = cfg()
  rules = c.logical_axis_rules
  # 'mlp' comes before 'embed' in the table and takes fsdp_transpose, so 'embed' falls back to its second rule
  got = R.logical_to_mesh_axes(("embed", "mlp"), rules)
  assert got[1][0] == "fsdp_transpose" and "fsdp_transpose" not in got[0] and got[0][0] == "fsdp"
  assert R.logical_to_mesh_axes(("nothing_here", None), rules) == [(), ()]
  assert R.logical_to_mesh_axes(("kv",), rules) == [()]


def test_size_one_axes_dropped_and_indivisible_dims_replicated():
  c = cfg("ici_fsdp_parallelism=4", "ici_tensor_parallelism=2")
  ms = dict(zip(c.mesh_axes, c.mesh_shape))
  s = R.make_spec(("embed", "mlp"), c.logical_axis_rules, ms, (4096, 14336))
  assert s.dims == (("fsdp",), ("tensor",)) and s.local_shape(ms) == (1024, 7168)
  s = R.make_spec(("embed", "mlp"), c.logical_axis_rules, ms, (4098, 14336))
  assert s.dims[0] == ()


def test_expert_axis_doubles_as_fsdp_for_dense_weights():
  c = cfg("ici_fsdp_parallelism=1", "ici_expert_parallelism=8", "model_name=mixtral-8x7b")
  ms = dict(zip(c.mesh_axes, c.mesh_shape))
  dense = R.make_spec(("embed", "mlp"), c.logical_axis_rules, ms, (4096, 14336))
  expert = R.make_spec(("exp", "embed_moe", "mlp_moe"), c.logical_axis_rules, ms, (8, 4096, 14336))
  assert dense.dims[0] == ("expert",) and expert.dims == (("expert",), (), ())


def test_sufficiently_sharded_assertion():
  ms = {"fsdp": 8}
  good = {"w": R.ShardSpec((("fsdp",), ()), (4096, 4096))}
  bad = {"w": R.ShardSpec(((), ()), (4096, 4096))}
  R.assert_params_sufficiently_sharded(good, ms, 0.02)
  with pytest.raises(AssertionError):
    R.assert_params_sufficiently_sharded(bad, ms, 0.02)


def test_mesh_coordinates_and_groups():
  m = Mesh(["data", "fsdp", "tensor"], [2, 2, 2], rank=5, world=8)
  assert m.coords == {"data": 1, "fsdp": 0, "tensor": 1}
  assert m.rank_of(m.coords) == 5
  assert m.ranks_along("tensor") == [4, 5] and m.ranks_along("fsdp") == [5, 7] and m.ranks_along(("data", "fsdp")) == [1, 3, 5, 7]
  assert m.axis_index(("data", "fsdp")) == 2 and m.axis_size(("fsdp", "tensor")) == 4


def _dump(model, overrides, n):
  import torch
  from maxtext_b200.models.transformer import Transformer
  c = cfg(f"model_name={model}", *overrides, n=n)
  mesh = Mesh(list(c.mesh_axes), list(c.mesh_shape), rank=0, world=n)
  model_obj = Transformer(c, mesh, torch.device("meta"), build_store=False)
  ms = mesh.shape
  out = {}
  for p in model_obj.all_params():
    d = p.pdef
    if d.layer not in (None, 0):
      continue
    out[d.name] = R.make_spec(d.logical_axes, c.logical_axis_rules, ms, d.ref_shape).to_json()
  return out


GOLDEN = os.path.join(ROOT, "tests", "golden", "sharding")
CASES = [("llama3-8b", ["ici_fsdp_parallelism=8"], 8, "llama3-8b_fsdp8"),
         ("llama3-70b", ["ici_fsdp_parallelism=4", "ici_tensor_parallelism=2"], 8, "llama3-70b_fsdp4_tp2"),
         ("mixtral-8x7b", ["ici_fsdp_parallelism=1", "ici_expert_parallelism=8"], 8, "mixtral-8x7b_ep8"),
         ("deepseek2-16b", ["ici_fsdp_parallelism=1", "ici_expert_parallelism=8"], 8, "deepseek2-16b_ep8")]


@pytest.mark.parametrize("model,over,n,tag", CASES)
def test_golden_sharding_dump(model, over, n, tag):
  got = _dump(model, over, n)
  path = os.path.join(GOLDEN, tag + ".json")
  if os.environ.get("UPDATE_GOLDEN") == "1" or not os.path.exists(path):
    os.makedirs(GOLDEN, exist_ok=True)
    json.dump(got, open(path, "w"), indent=1, sort_keys=True)
  want = json.load(open(path))
  assert got == want
