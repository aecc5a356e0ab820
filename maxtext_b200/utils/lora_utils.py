"""LoRA adapters: merge / un-merge into the base weights, and HF-PEFT adapter files.

Counterpart of src/maxtext/utils/lora_utils.py (`apply_lora_on_base_params` 61, `unapply_lora_from_base_params` 101,
`load_adapter` 141). Adapters are created by `layers.blocks.Builder.linear` when `lora.enable_lora` is set: for a
linear with weight W [out, in] the model computes W x + (alpha / r) B (A x) with A [r, in] and B [out, r], and every
other parameter is frozen. Serving usually wants one plain weight instead: `merge` adds (alpha / r) B A into the fp32
master of W (and `unmerge` subtracts it again), after which a model built without adapters gives the same outputs.

Adapter files follow the PEFT layout (`adapter_config.json` + `adapter_model.safetensors`, keys
`base_model.model.<hf module>.lora_A.weight` / `.lora_B.weight`), with the same per-family transforms as the
checkpoint converter: the query scale folded into B of the query projection and the rotary lane permutation applied
to the output rows of the query / key adapters.
"""
from __future__ import annotations

import json
import os

import torch

from ..checkpoint_conversion import hf as conv


def adapted(store):
  """[(base param, A, B, scale)] for every linear that carries an adapter."""
  return [(p,) + tuple(p.lora) for p in store.params.values() if getattr(p, "lora", None) is not None]


def _delta(store, a, b, scale) -> torch.Tensor:
  return (store.full_master(b).float() @ store.full_master(a).float()) * scale


def merge(store, sign: float = 1.0):
  """W <- W + sign * (alpha / r) B A for every adapted linear (collective over each unit's shard group)."""
  for p, a, b, scale in adapted(store):
    w = store.full_master(p).float() + sign * _delta(store, a, b, scale).view(p.pdef.global_shape())
    store.load_full(p.name, p.pdef.local_slice(w))
  store.sync_compute_from_master()


def unmerge(store):
  merge(store, -1.0)


def merged_base_state(store) -> dict:
  """{base parameter name: merged fp32 weight}: what a model without adapters has to load to behave like this one."""
  return {p.name: store.full_master(p).float() + _delta(store, a, b, scale).view(p.pdef.global_shape())
          for p, a, b, scale in adapted(store)}


# ------------------------------------------------------------------------------------------ PEFT files
def _peft_key(p, cfg) -> tuple[str, str] | None:
  m = conv._hf_name(p.pdef, cfg)  # pylint: disable=protected-access
  if m is None or not m[0].endswith(".weight"):
    return None
  return "base_model.model." + m[0][:-len(".weight")], m[1]


def to_peft(store, cfg) -> tuple[dict, dict]:
  """(state dict, adapter_config) in PEFT conventions."""
  out, modules = {}, set()
  inter = conv._interleaved(cfg)  # pylint: disable=protected-access
  rank, alpha = None, None
  for p, a, b, scale in adapted(store):
    k = _peft_key(p, cfg)
    if k is None:
      continue
    key, kind = k
    A, B = store.full_master(a).float().clone(), store.full_master(b).float().clone()
    rank, alpha = A.shape[0], scale * A.shape[0]
    if kind == "q":
      B = B / conv._q_scale(cfg)  # pylint: disable=protected-access
      if inter:
        B = conv._deinterleave(B, cfg.num_query_heads, cfg.head_dim)  # pylint: disable=protected-access
    elif kind == "k" and inter:
      B = conv._deinterleave(B, cfg.num_kv_heads, cfg.head_dim)  # pylint: disable=protected-access
    out[key + ".lora_A.weight"], out[key + ".lora_B.weight"] = A.contiguous(), B.contiguous()
    modules.add(key.rsplit(".", 1)[1])
  acfg = {"peft_type": "LORA", "r": rank, "lora_alpha": alpha, "target_modules": sorted(modules), "bias": "none",
          "task_type": "CAUSAL_LM", "lora_dropout": 0.0}
  return out, acfg


def from_peft(state: dict, store, cfg) -> list[str]:
  """Load PEFT tensors into the adapters; returns the adapted linears that had no tensors in `state`."""
  inter = conv._interleaved(cfg)  # pylint: disable=protected-access
  missing = []
  for p, a, b, _ in adapted(store):
    k = _peft_key(p, cfg)
    ka = (k[0] + ".lora_A.weight") if k else None
    if k is None or ka not in state:
      ka2 = (k[0] + ".lora_A.default.weight") if k else None       # in-memory PEFT models name the adapter
      if k is None or ka2 not in state:
        missing.append(p.name)
        continue
      ka, kb = ka2, k[0] + ".lora_B.default.weight"
    else:
      kb = k[0] + ".lora_B.weight"
    A, B = state[ka].float(), state[kb].float()
    kind = k[1]
    if kind == "q":
      if inter:
        B = conv._interleave(B, cfg.num_query_heads, cfg.head_dim)  # pylint: disable=protected-access
      B = B * conv._q_scale(cfg)  # pylint: disable=protected-access
    elif kind == "k" and inter:
      B = conv._interleave(B, cfg.num_kv_heads, cfg.head_dim)  # pylint: disable=protected-access
    assert tuple(A.shape) == tuple(a.pdef.global_shape()), (p.name, A.shape, a.pdef.global_shape())
    store.load_full(a.name, a.pdef.local_slice(A.contiguous()))
    store.load_full(b.name, b.pdef.local_slice(B.contiguous()))
  store.sync_compute_from_master()
  return missing


def save_adapter(directory: str, store, cfg):
  from safetensors.torch import save_file
  state, acfg = to_peft(store, cfg)
  os.makedirs(directory, exist_ok=True)
  save_file(state, os.path.join(directory, "adapter_model.safetensors"))
  with open(os.path.join(directory, "adapter_config.json"), "w") as fh:
    json.dump(acfg, fh, indent=1)
  return directory


def load_adapter(directory: str, store, cfg) -> dict:
  """Read a PEFT adapter directory into the model's adapters; returns its adapter_config. The model must have been built
  with the same rank (and target modules at least as wide) as the file."""
  from safetensors.torch import load_file
  with open(os.path.join(directory, "adapter_config.json")) as fh:
    acfg = json.load(fh)
  missing = from_peft(load_file(os.path.join(directory, "adapter_model.safetensors")), store, cfg)
  if missing and len(missing) == len(adapted(store)):
    raise KeyError(f"no adapter tensors for any adapted linear, e.g. {missing[:3]}")
  return acfg
