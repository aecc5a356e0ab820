"""Weights for a vLLM engine (src/maxtext/integration/vllm/{weight_converter,convert_utils}.py).

vLLM models load weights through `model.load_weights(iterable of (hf_name, tensor))` with HuggingFace names and layouts
(they fuse q|k|v and gate|up themselves). `weights_iterator` produces exactly that stream from a ParamStore, one
parameter at a time (a collective over the parameter's shard group, so every rank of the trainer calls it), which is
what an RL loop needs to push fresh policy weights into its rollout engine without writing a checkpoint:

    llm.llm_engine.model_executor.driver_worker.model_runner.model.load_weights(weights_iterator(engine.store, cfg))

`sync_weights` does that call for an in-process `vllm.LLM`; `rollout` wraps generation with sampling parameters and
returns token ids and log-probabilities in the shape the GRPO trainer of `trainers/post_train` consumes.
"""
from __future__ import annotations

from typing import Iterator

import torch

from ..checkpoint_conversion import hf as conv


def weights_iterator(store, cfg, dtype: torch.dtype | None = None) -> Iterator[tuple[str, torch.Tensor]]:
  """(HF name, tensor) pairs for every parameter that has an HF counterpart; stacked experts are emitted per expert."""
  if conv._expert_style(cfg) in ("gpt_oss", "llama4"):  # pylint: disable=protected-access
    # these families store gate and up of all experts in one HF tensor assembled from two of ours: export in one piece
    for k, v in conv.to_hf(store, cfg).items():
      yield k, (v.to(dtype) if dtype is not None else v)
    return
  for p in store.params.values():
    m = conv._hf_name(p.pdef, cfg)  # pylint: disable=protected-access
    if m is None:
      continue
    one = conv.to_hf(_Single(store, p), cfg)       # reuse the exporter's per-kind transforms for this one parameter
    for k, v in one.items():
      yield k, (v.to(dtype) if dtype is not None else v)


class _Single:
  """A store view that exposes one parameter (what `to_hf` iterates over)."""

  def __init__(self, store, p):
    self._store, self.params = store, {p.name: p}

  def full_master(self, p):
    return self._store.full_master(p)


def _vllm_model(llm):
  ex = llm.llm_engine.model_executor
  return ex.driver_worker.model_runner.model


def sync_weights(llm, store, cfg, dtype: torch.dtype = torch.bfloat16) -> int:
  """Load the trainer's current weights into an in-process `vllm.LLM`; returns how many tensors were sent."""
  n = 0

  def counted():
    nonlocal n
    for item in weights_iterator(store, cfg, dtype):
      n += 1
      yield item
  _vllm_model(llm).load_weights(counted())
  return n


def rollout(llm, prompt_token_ids: list[list[int]], max_new_tokens: int, temperature: float = 1.0, top_p: float = 1.0, n: int = 1):
  """Sample `n` completions per prompt; returns [(prompt index, token ids, per-token log-probabilities)]."""
  from vllm import SamplingParams
  sp = SamplingParams(max_tokens=int(max_new_tokens), temperature=float(temperature), top_p=float(top_p), n=int(n), logprobs=0)
  outs = llm.generate([{"prompt_token_ids": ids} for ids in prompt_token_ids], sp)
  res = []
  for i, o in enumerate(outs):
    for c in o.outputs:
      lps = [next(iter(d.values())).logprob for d in (c.logprobs or [])]
      res.append((i, list(c.token_ids), lps))
  return res
