"""Ahead-of-time plan of a training job: `python -m maxtext_b200.train.train_compile <yml> compile_topology=b200-8 key=value ...`.

The role of src/maxtext/trainers/pre_train/train_compile.py (AOT-compile `train_step` for a topology that is not
attached and report whether it fits): nothing is traced here, so the "compiled artefact" is the plan the engine will
execute -- parameter units and their shard groups, what each rank holds, what moves over NVLink per step -- plus a
memory estimate against the HBM of the target part and a roofline step-time estimate. The model is built on the meta
device with the mesh of the *target* world, so no GPU and no process group is needed; `compiled_trainstep_file`
receives the plan as JSON.
"""
from __future__ import annotations

import json
import re
import sys

from ..config import pyconfig
from ..layers.context import saved_names
from ..parallel import mesh as mesh_lib
from ..utils import flops as flops_lib
from ..utils import max_logging

HBM_BYTES = {"b200": 180e9, "h100": 80e9, "h200": 141e9, "a100": 80e9}
PEAK = {"b200": dict(tflops=1400.0, hbm_gbs=6650.0, nvlink_gbs=770.0)}   # sustained bf16 GEMM, copy bandwidth, peer copy per direction


def parse_topology(topo: str, num_slices: int = 1) -> tuple[str, int]:
  """'b200-8' -> ('b200', 8); slices multiply the device count (compile_topology_num_slices)."""
  m = re.fullmatch(r"([a-z0-9]+?)-(\d+)", topo.strip().lower())
  if not m:
    raise ValueError(f"compile_topology must look like b200-8, got {topo!r}")
  return m.group(1), int(m.group(2)) * max(1, num_slices)


def _saved_bytes_per_token(c, names) -> float:
  """Bytes per token and layer kept by the remat policy, beside the layer input (bf16)."""
  hq, hkv, dh, e, f = c.num_query_heads, c.num_kv_heads, c.head_dim, c.emb_dim, c.mlp_dim
  size = {"query_proj": hq * dh, "key_proj": hkv * dh, "value_proj": hkv * dh, "qkv_proj": (hq + 2 * hkv) * dh, "kv_proj": 2 * hkv * dh,
          "out_proj": e, "context": hq * dh, "mlpwi_0": f, "mlpwi_1": f, "mlpwi": 2 * f, "mlpwo": e}
  fused = {"qkv_proj": ("query_proj", "key_proj", "value_proj"), "mlpwi": ("mlpwi_0", "mlpwi_1"), "kv_proj": ("key_proj", "value_proj")}
  names = set(names)
  for whole, parts in fused.items():       # a fused projection is stored once
    if whole in names:
      names -= set(parts)
  return 2.0 * sum(size.get(n, 0) for n in names)


def plan(config, world: int | None = None, part: str = "b200") -> dict:
  from ..models.transformer import Transformer
  c = config
  world = world or c.num_target_devices
  mesh = mesh_lib.mesh_from_config(c, rank=0, world=world) if world > 1 else None
  model = Transformer(c, mesh, "meta")
  st = model.store
  tp = model.par["tp_size"]
  cp = mesh.axis_size("context") if mesh is not None else 1
  units = []
  for name, u in st.units.items():
    units.append(dict(name=name, numel=int(u.numel), shard_numel=int(u.chunk), shard_group=int(u.group_size),
                      params=[p.name for p in u.params][:4] + (["..."] if len(u.params) > 4 else [])))
  local = int(st.master.numel())
  wbytes = 2 if str(c.weight_dtype) in ("bfloat16", "float16") else 4
  # ---- per-rank state
  opt_states = {"adamw": 2, "adam_pax": 2, "sgd": 0, "muon": 1}.get(c.opt_type, 2)
  mem = {}
  mem["master_weights"] = local * wbytes
  mem["compute_shard_bf16"] = 0 if (wbytes == 2 and c.dtype == "bfloat16") else local * 2
  mu_bytes = 2 if str(getattr(c, "mu_dtype", "") or c.weight_dtype) in ("bfloat16", "float16") else 4
  # first moment in mu_dtype, second moment always fp32
  mem["optimizer_state"] = local * (mu_bytes + 4 * (opt_states - 1)) if opt_states >= 1 else 0
  mem["grad_shard_fp32"] = local * 4
  sharded = [u for u in st.units.values() if u.group_size > 1]
  max_unit = max((u.numel for u in sharded), default=0)
  n_buf = 2 + int(c.fsdp_prefetch_units)
  mem["gathered_unit_buffers"] = n_buf * max_unit * 2
  mem["full_grad_buffers_fp32"] = 2 * max_unit * 4
  # ---- activations
  B = c.per_device_batch_size
  S = c.max_target_length / max(1, cp)
  tok = B * S
  L = len(model.layers)
  dev_names, off_names = saved_names(c)
  mem["layer_input_checkpoints"] = L * tok * c.emb_dim * 2
  mem["remat_saved"] = L * tok * _saved_bytes_per_token(c, dev_names) / tp
  host_offload = L * tok * _saved_bytes_per_token(c, off_names) / tp
  # live set of one layer under autograd (recompute + backward): projections, context, gate/up/act, norms, fp32 softmax stats
  f_loc = (c.mlp_dim if c.num_experts <= 1 else c.mlp_dim * c.num_experts_per_tok * c.capacity_factor if c.capacity_factor > 0
           else c.mlp_dim * c.num_experts_per_tok) / tp
  per_tok = 2.0 * (4 * c.emb_dim + (2 * c.num_query_heads + 2 * c.num_kv_heads) * c.head_dim / tp + 4 * f_loc)
  mem["one_layer_live_activations"] = tok * per_tok * 2          # forward tensors + their gradients
  chunk = c.head_chunk_tokens if getattr(c, "head_chunk_tokens", 0) > 0 else min(tok, 8192)
  mem["head_logits_chunk"] = min(tok, chunk) * (c.vocab_size / tp) * (4 + 2)
  total = float(sum(mem.values()))
  hbm = HBM_BYTES.get(part, 180e9)
  # ---- traffic and time
  fsdp_bytes = sum(u.numel for u in sharded)
  ag = 2 * fsdp_bytes * 2 * (1 - 1 / max(1, max((u.group_size for u in sharded), default=1)))   # forward + recompute gathers, bf16
  rs = fsdp_bytes * 4 * (1 - 1 / max(1, max((u.group_size for u in sharded), default=1)))
  tfl, _, _ = flops_lib.training_tflops_per_device(c)
  recompute = 4.0 / 3.0 if c.remat_policy == "full" else 1.0
  pk = PEAK.get(part, PEAK["b200"])
  t_compute = tfl * recompute / pk["tflops"]
  t_comm = (ag + rs) / (pk["nvlink_gbs"] * 1e9)
  t_opt = local * (4 * 4 + 4 * 3 + 2) / (pk["hbm_gbs"] * 1e9)
  out = dict(
      model=c.model_name, part=part, world=world, mesh={a: mesh.axis_size(a) for a in mesh.axis_names} if mesh is not None else {},
      parameters_total=int(st.num_parameters()), parameters_per_rank=local, units=units,
      memory_bytes={k: int(v) for k, v in mem.items()}, memory_total_gb=round(total / 1e9, 2), hbm_gb=hbm / 1e9,
      host_offload_gb=round(host_offload / 1e9, 2), fits=bool(total < 0.94 * hbm),
      per_step=dict(model_tflops_per_device=round(tfl, 1), executed_tflops_per_device=round(tfl * recompute, 1),
                    all_gather_bytes=int(ag), reduce_scatter_bytes=int(rs),
                    est_compute_s=round(t_compute, 4), est_comm_s=round(t_comm, 4), est_optimizer_s=round(t_opt, 4),
                    est_step_s=round(max(t_compute, t_comm) + t_opt, 4),
                    est_tokens_per_s_per_device=round(tok / (max(t_compute, t_comm) + t_opt), 1)))
  return out


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  topo = next((a.split("=", 1)[1] for a in argv if a.startswith("compile_topology=")), "")
  slices = next((int(a.split("=", 1)[1]) for a in argv if a.startswith("compile_topology_num_slices=")), 1)
  part, world = parse_topology(topo, slices) if topo else ("b200", None)
  config = pyconfig.initialize(argv, num_devices=world)
  p = plan(config, world or config.num_target_devices, part)
  max_logging.log(json.dumps({k: v for k, v in p.items() if k != "units"}, indent=1))
  if config.compiled_trainstep_file:
    with open(config.compiled_trainstep_file, "w") as fh:
      json.dump(p, fh, indent=1)
  if not p["fits"]:
    max_logging.log(f"DOES NOT FIT: {p['memory_total_gb']} GB needed of {p['hbm_gb']} GB")
    return 1
  return 0


if __name__ == "__main__":
  sys.exit(main())
