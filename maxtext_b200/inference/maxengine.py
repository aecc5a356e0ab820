"""Decode engine with the MaxEngine API shape: load_params / prefill / insert / generate / init_decode_state
(src/maxtext/inference/maxengine/maxengine.py:114-1933).

State lives in `DecodeState`: per-layer KV caches with `slots` rows, the last sampled token and the next position of
every slot. `prefill` runs one prompt through the model into a private single-row cache and samples the first
token; `insert` copies that cache into a slot of the decode state; `generate` advances every active slot by one
token. All units of the model must be resident (single GPU, or tensor-parallel ranks each holding their slice).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import os

import torch

from ..models.transformer import Transformer
from . import inference_utils, kvcache


@dataclass
class Prefix:
  caches: list
  length: int
  first_token: torch.Tensor       # [1]
  logits: torch.Tensor            # [1, V] logits at the last prompt position
  log_prob: torch.Tensor | None = None


@dataclass
class DecodeState:
  caches: list
  tokens: torch.Tensor            # [slots] last sampled token per slot
  next_pos: torch.Tensor          # [slots] position the next token will be written at (= cached length)
  active: torch.Tensor            # [slots] bool
  generated: torch.Tensor         # [slots] tokens generated so far
  token_logp: torch.Tensor | None = None


@dataclass
class ResultTokens:
  data: torch.Tensor              # [slots, 3] = token, valid flag, generated length
  log_prob: torch.Tensor | None = None


class MaxEngine:
  def __init__(self, config, mesh=None, device=None, model: Transformer | None = None):
    self.config = c = config
    if device is None:
      device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and c.hardware != "cpu" else "cpu"
    self.device = torch.device(device)
    self.model = model or Transformer(c, mesh, self.device)
    self.max_len = int(c.max_target_length)
    # a prompt must leave room for at least one generated token (prefill / insert check every length against max_len - 1);
    # training configs that build a sampler keep the default prefill length, so it is capped here rather than refused
    self.max_prefill = min(int(c.max_prefill_predict_length), self.max_len - 1)
    self.generator = torch.Generator(device=self.device)
    self.generator.manual_seed(int(c.init_weights_seed))
    self._graphs: dict = {}          # id(state) -> (CUDAGraph, static result tensors) when cuda_graphs is on

  # ------------------------------------------------------------------ params
  def load_params(self, path: str | None = None, seed: int | None = None):
    """Params-only checkpoint (`load_parameters_path`) or random init when no path is configured."""
    from ..checkpoint import manager as ckpt
    path = path or self.config.load_parameters_path
    if path:
      ckpt.load_params_only(path, _EngineView(self), self.model.mesh)
    else:
      self.model.store.initialize(seed=self.config.init_weights_seed if seed is None else seed)
    c = self.config
    if bool(getattr(c, "checkpoint_is_quantized", False)) and path and os.path.isfile(os.path.join(path, "quantized_params.safetensors")):
      self.load_quantized_params(os.path.join(path, "quantized_params.safetensors"))
    elif str(getattr(c, "quantization", "") or "") in ("int8", "int4", "intmp") and str(getattr(c, "save_quantized_params_path", "") or ""):
      # serving flow of the reference (maxengine.py:576-620): quantise the loaded weights once and write them out
      self.save_quantized_params(c.save_quantized_params_path, 8 if c.quantization == "int8" else 4)
    return self.model.store

  def save_quantized_params(self, directory: str, bits: int = 8) -> str:
    from safetensors.torch import save_file
    packed = self.quantize_params(bits)
    flat = {}
    for n, (q, sc) in packed.items():
      flat[n + "/q"], flat[n + "/scale"] = q.contiguous(), sc.contiguous()
    os.makedirs(directory, exist_ok=True)
    out = os.path.join(directory, "quantized_params.safetensors")
    save_file(flat, out)
    return out

  @torch.no_grad()
  def load_quantized_params(self, file: str):
    """`checkpoint_is_quantized`: matrices come from (int values, per-channel scales); the rest keeps its loaded value."""
    from safetensors.torch import load_file
    flat = load_file(file)
    store = self.model.store
    for name, p in store.params.items():
      if name + "/q" in flat:
        q, sc = flat[name + "/q"].float(), flat[name + "/scale"].float()
        if sc.dim() == q.dim():                  # sub-channel scales [..., out, tiles]: one per stretch of the contraction dim
          sc = sc.repeat_interleave(q.shape[-1] // sc.shape[-1], dim=-1)
          w = q * sc
        else:
          w = q * sc[..., None]
        store.load_full(name, p.pdef.local_slice(w))
    store.sync_compute_from_master()

  # ------------------------------------------------------------------ state
  @torch.no_grad()
  def quantize_params(self, bits: int = 8, mixed=None) -> dict:
    """Weight-only quantisation for serving (src/maxtext/inference/maxengine/maxengine.py:576 `quantize_params`): every
    matrix inside the decoder layers is rounded to `bits`-bit integers with one scale per output channel, or per matrix as a
    mixed-precision map says (`mixed` = `mixed_precision.load_quant_map(path)`; `quantization=intmp` loads `quant_cfg_path`).
    Returns {name: (int8 values, fp32 scales)} for saving; the engine's own weights are replaced by the de-quantised values,
    so what it generates afterwards is what a server loading the quantised file generates (it still computes in bf16)."""
    from . import mixed_precision as mp
    store = self.model.store
    c = self.config
    if mixed is None and str(getattr(c, "quantization", "") or "") == "intmp":
      if not str(getattr(c, "quant_cfg_path", "") or ""):
        raise ValueError("quantization=intmp needs quant_cfg_path")
      mixed = mp.load_quant_map(c.quant_cfg_path)
    packed = {}
    for name, p in store.params.items():
      d = p.pdef
      if d.layer is None or d.kind not in ("linear", "expert_linear") or len(d.shape) < 2:
        continue
      cfg = mp.settings_for(name, mixed) if mixed is not None else {"w_bits": int(bits), "tile_size": -1, "w_scale": 1.0}
      q, scale, deq = mp.quantize_weight(store.full_master(p).float(), cfg)
      packed[name] = (q, scale)
      store.load_full(name, d.local_slice(deq))
    store.sync_compute_from_master()
    return packed

  def init_decode_state(self, slots: int | None = None) -> DecodeState:
    c = self.config
    slots = int(slots or max(1, int(c.per_device_batch_size)))
    dev = self.device
    return DecodeState(kvcache.make_caches(self.model, slots, self.max_len, dev), torch.zeros(slots, dtype=torch.long, device=dev),
                       torch.zeros(slots, dtype=torch.long, device=dev), torch.zeros(slots, dtype=torch.bool, device=dev),
                       torch.zeros(slots, dtype=torch.long, device=dev),
                       torch.zeros(slots, device=dev) if c.return_log_prob else None)

  def _bind(self, caches, slot_ids, lengths):
    for per_layer in caches:
      for cch in per_layer:
        cch.bind(slot_ids, lengths)

  def _check_length(self, n: int, what: str):
    """A prompt must leave room for at least one generated token: a prefix of max_target_length tokens would make the next
    decode step write its key / value one row past the end of the slot's cache."""
    n = int(n)
    if n < 1 or n >= self.max_len:
      raise ValueError(f"{what}: length {n} is outside [1, max_target_length - 1 = {self.max_len - 1}]")

  def _sample(self, logits):
    c = self.config
    return inference_utils.sampling(logits, c.decode_sampling_strategy, int(c.decode_sampling_top_k), float(c.decode_sampling_nucleus_p),
                                    float(c.decode_sampling_temperature), self.generator)

  # ------------------------------------------------------------------ prefill / insert / generate
  @torch.no_grad()
  def prefill(self, padded_tokens: torch.Tensor, true_length: int, params=None, images=None, image_mask=None, audio=None,
              audio_mask=None) -> tuple[Prefix, ResultTokens]:
    """padded_tokens [P] (right padded); only the first `true_length` enter the cache. `images` [N, 3, H, W] with
    `image_mask` [P] (True at the soft-token positions of the prompt) makes the prompt multimodal; `audio` [mel, frames] (one
    clip) with `audio_mask` [P] does the same for the audio tower."""
    dev = self.device
    self._check_length(true_length, "prefill")
    if int(true_length) > int(padded_tokens.numel()):
      raise ValueError(f"prefill: true_length {true_length} exceeds the {int(padded_tokens.numel())} tokens given")
    toks = padded_tokens[:true_length].to(dev).long()[None]
    caches = kvcache.make_caches(self.model, 1, max(self.max_prefill, true_length), dev)
    self._bind(caches, torch.zeros(1, dtype=torch.long, device=dev), torch.zeros(1, dtype=torch.long, device=dev))
    pos = torch.arange(true_length, device=dev)[None]
    mm_kw = {}
    if images is not None:
      mm_kw = dict(images=images[None].to(dev), image_mask=image_mask[:true_length][None].to(dev))
    if audio is not None:
      mm_kw.update(audio=audio[None].to(dev), audio_mask=audio_mask[:true_length][None].to(dev))
    logits = self.model.forward(toks, pos, None, mode="prefill", caches=caches, **mm_kw)[:, -1]
    tok = self._sample(logits)
    lp = inference_utils.log_prob_of(logits, tok) if self.config.return_log_prob else None
    res = ResultTokens(torch.tensor([[int(tok), 1, 1]], device=dev), lp)
    return Prefix(caches, true_length, tok, logits, lp), res

  @torch.no_grad()
  def prefill_multisampling(self, padded_tokens: torch.Tensor, true_length: int, num_samples: int):
    """One prefill pass, `num_samples` independently sampled first tokens (src/maxtext/inference/maxengine/maxengine.py:998-1180):
    the prefixes share the cached prompt and differ in their first token, e.g. for best-of-n or GRPO-style rollouts."""
    prefix, _ = self.prefill(padded_tokens, true_length)
    out = []
    for _ in range(int(num_samples)):
      tok = self._sample(prefix.logits)
      lp = inference_utils.log_prob_of(prefix.logits, tok) if self.config.return_log_prob else None
      out.append(Prefix(prefix.caches, prefix.length, tok, prefix.logits, lp))
    return out

  @torch.no_grad()
  def prefill_concat(self, prompts: list[torch.Tensor]) -> list[Prefix]:
    """Several short prompts in one prefill pass (maxengine.py:1180 `prefill_concat`): the prompts are packed into one row
    with segment ids and per-prompt positions, and the cached keys / values of each segment become that prompt's prefix.
    Layers with a recurrent state (gated delta networks) cannot be packed this way; such models prefill one by one."""
    dev = self.device
    lens = [int(p.numel()) for p in prompts]
    for n in lens:
      self._check_length(n, "prefill_concat")
    total = sum(lens)
    packable = total <= self.max_len and not any(b.plan.attention in ("gdn", "compressed") for l in self.model.layers for b in l.blocks)
    if not packable or len(prompts) == 1:
      return [self.prefill(p, n)[0] for p, n in zip(prompts, lens)]
    toks = torch.cat([p.to(dev).long() for p in prompts])[None]
    seg = torch.cat([torch.full((n,), i + 1, dtype=torch.int32, device=dev) for i, n in enumerate(lens)])[None]
    pos = torch.cat([torch.arange(n, device=dev) for n in lens])[None]
    packed = kvcache.make_caches(self.model, 1, total, dev)
    zero = torch.zeros(1, dtype=torch.long, device=dev)
    self._bind(packed, zero, zero)
    logits = self.model.forward(toks, pos, seg, mode="prefill", caches=packed)[0]
    out, start = [], 0
    for n in lens:
      caches = kvcache.make_caches(self.model, 1, max(self.max_prefill, n), dev)
      for dst_layer, src_layer in zip(caches, packed):
        for d, s_ in zip(dst_layer, src_layer):
          for name in ("k", "v", "ks", "vs", "latent", "k_rope"):
            if hasattr(s_, name) and hasattr(d, name):
              getattr(d, name)[0, :n] = getattr(s_, name)[0, start:start + n]
      lg = logits[start + n - 1][None]
      tok = self._sample(lg)
      out.append(Prefix(caches, n, tok, lg, inference_utils.log_prob_of(lg, tok) if self.config.return_log_prob else None))
      start += n
    return out

  @torch.no_grad()
  def bulk_insert(self, prefix: Prefix, state: DecodeState, slots: list[int]) -> DecodeState:
    """The same prefix into several slots (maxengine.py:1477), e.g. the prefixes of `prefill_multisampling` share a prompt."""
    for s in slots:
      state = self.insert(prefix, state, int(s))
    return state

  def prefill_chunked(self, tokens: torch.Tensor, chunk: int | None = None) -> tuple[Prefix, ResultTokens]:
    """Chunked prefill (src/maxtext/inference/kvcache.py:609-712): the prompt enters the cache `chunk` tokens at a time."""
    dev = self.device
    chunk = int(chunk or self.config.prefill_chunk_size)
    n = int(tokens.numel())
    self._check_length(n, "prefill_chunked")
    caches = kvcache.make_caches(self.model, 1, max(self.max_prefill, n), dev)
    slot = torch.zeros(1, dtype=torch.long, device=dev)
    logits = None
    with torch.no_grad():
      for s in range(0, n, chunk):
        e = min(n, s + chunk)
        self._bind(caches, slot, torch.full((1,), s, dtype=torch.long, device=dev))
        pos = torch.arange(s, e, device=dev)[None]
        logits = self.model.forward(tokens[s:e].to(dev).long()[None], pos, None, mode="decode", caches=caches)[:, -1]
    tok = self._sample(logits)
    return Prefix(caches, n, tok, logits), ResultTokens(torch.tensor([[int(tok), 1, 1]], device=dev))

  @torch.no_grad()
  def insert(self, prefix: Prefix, state: DecodeState, slot: int) -> DecodeState:
    n = prefix.length
    self._check_length(n, "insert")
    if not 0 <= int(slot) < int(state.tokens.shape[0]):
      raise ValueError(f"insert: slot {slot} is outside [0, {int(state.tokens.shape[0])})")
    for dst_layer, src_layer in zip(state.caches, prefix.caches):
      for d, s in zip(dst_layer, src_layer):
        m = s.rows_for(n) if hasattr(s, "rows_for") else n          # rows of this rank's part of a sequence-split cache
        for name in ("k", "v", "ks", "vs", "latent", "k_rope") + tuple(getattr(s, "token_buffers", ())):
          if hasattr(s, name) and hasattr(d, name):
            getattr(d, name)[slot, :m] = getattr(s, name)[0, :m]
        for name in ("conv", "rec"):                 # fixed-size recurrent state (gated delta layers)
          if hasattr(s, name) and hasattr(d, name):
            getattr(d, name)[slot] = getattr(s, name)[0]
    state.tokens[slot] = prefix.first_token.reshape(-1)[0]
    state.next_pos[slot] = n
    state.active[slot] = True
    state.generated[slot] = 1
    return state

  @torch.no_grad()
  def generate(self, state: DecodeState, params=None) -> tuple[DecodeState, ResultTokens]:
    """One autoregressive step for every slot (inactive slots compute too; their results are flagged invalid).

    With `cuda_graphs=true` on a GPU the step is captured once per decode state and replayed: a decode step is a few
    hundred small launches, so replaying one graph removes the launch latency that otherwise dominates it. The state
    tensors are updated in place (the graph reads and writes fixed addresses); everything data-dependent (lengths, slot
    ids, sampling) stays on the device."""
    if self.device.type == "cuda" and bool(getattr(self.config, "cuda_graphs", False)):
      out = self._generate_graphed(state)
      if out is not None:
        return out
    return self._generate_eager(state)

  def _step_inplace(self, state: DecodeState):
    """The decode step with every state update written into the existing tensors."""
    dev = self.device
    slots = state.tokens.shape[0]
    ids = torch.arange(slots, device=dev)
    self._bind(state.caches, ids, state.next_pos.clone())
    logits = self.model.forward(state.tokens[:, None], state.next_pos[:, None], None, mode="decode", caches=state.caches)[:, -1]
    tok = self._sample(logits)
    if state.token_logp is not None:
      state.token_logp.copy_(inference_utils.log_prob_of(logits, tok))
    state.tokens.copy_(torch.where(state.active, tok, state.tokens))
    state.next_pos.add_(state.active.long())
    state.generated.add_(state.active.long())
    data = torch.stack([state.tokens, state.active.long(), state.generated], dim=1)
    state.active.logical_and_(state.next_pos < self.max_len - 1)
    return data

  def _generate_graphed(self, state: DecodeState):
    key = id(state)
    entry = self._graphs.get(key)
    if entry is None:
      try:
        keep = [t.clone() for t in (state.tokens, state.next_pos, state.active, state.generated)]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                       # warm-up: lazy initialisation must happen outside the capture
          for _ in range(2):
            self._step_inplace(state)
        torch.cuda.current_stream().wait_stream(side)
        for t, k in zip((state.tokens, state.next_pos, state.active, state.generated), keep):
          t.copy_(k)                                        # the warm-up steps wrote only beyond the cached lengths
        g = torch.cuda.CUDAGraph()
        if hasattr(g, "register_generator_state"):
          g.register_generator_state(self.generator)
        with torch.cuda.graph(g):
          data = self._step_inplace(state)
        for t, k in zip((state.tokens, state.next_pos, state.active, state.generated), keep):
          t.copy_(k)                                        # capture does not execute, but keep the contract explicit
        entry = (g, data)
      except Exception as e:  # pylint: disable=broad-except
        from ..utils import max_logging
        max_logging.log(f"decode graph capture failed ({e!r}); running eagerly")
        entry = False
      self._graphs[key] = entry
    if entry is False:
      return None
    g, data = entry
    g.replay()
    return state, ResultTokens(data.clone(), state.token_logp)

  def _generate_eager(self, state: DecodeState) -> tuple[DecodeState, ResultTokens]:
    dev = self.device
    slots = state.tokens.shape[0]
    ids = torch.arange(slots, device=dev)
    self._bind(state.caches, ids, state.next_pos.clone())
    logits = self.model.forward(state.tokens[:, None], state.next_pos[:, None], None, mode="decode", caches=state.caches)[:, -1]
    tok = self._sample(logits)
    if state.token_logp is not None:
      state.token_logp = inference_utils.log_prob_of(logits, tok)
    state.tokens = torch.where(state.active, tok, state.tokens)
    state.next_pos = state.next_pos + state.active.long()
    state.generated = state.generated + state.active.long()
    full = state.next_pos >= self.max_len - 1
    res = ResultTokens(torch.stack([state.tokens, state.active.long(), state.generated], dim=1), state.token_logp)
    state.active = state.active & ~full
    return state, res

  def free_slot(self, state: DecodeState, slot: int):
    state.active[slot] = False
    state.next_pos[slot] = 0
    state.generated[slot] = 0


class _EngineView:
  """Adapter so checkpoint loading can treat an inference engine like a train engine."""

  def __init__(self, eng: MaxEngine):
    self.store, self.config, self.model = eng.model.store, eng.config, eng.model
    self.optimizer = type("NoOpt", (), {"state_arrays": staticmethod(lambda: {})})()
    self.step_count = 0
    self.device = eng.device
