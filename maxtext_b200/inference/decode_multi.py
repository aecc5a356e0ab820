"""`python -m maxtext_b200.inference.decode_multi <config.yml> prompts="a|b|c"`: several prompt streams through one engine
(src/maxtext/inference/decode_multi.py): prompts are prefilled (packed into one pass when the model allows), inserted into
free slots as they become available, and decoded together; finished streams free their slot for the next prompt."""
from __future__ import annotations

import sys

import torch

from ..config import pyconfig
from ..input_pipeline.tokenizer import build_tokenizer
from .maxengine import MaxEngine


def decode_multi(config, prompts: list[str], engine: MaxEngine | None = None, max_new_tokens: int | None = None) -> list[str]:
  eng = engine or MaxEngine(config)
  if engine is None:
    eng.load_params()
  tok = build_tokenizer(config)
  lim = int(config.max_prefill_predict_length)
  ids = [[i % config.vocab_size for i in tok.encode(p, add_bos=bool(config.add_bos))][-lim:] or [0] for p in prompts]
  budget = int(max_new_tokens or (int(config.max_target_length) - lim))
  slots = min(len(ids), int(getattr(config, "decode_slots", 0) or 4))
  state = eng.init_decode_state(slots=slots)
  prefixes = eng.prefill_concat([torch.tensor(t) for t in ids]) if sum(map(len, ids)) <= lim else \
      [eng.prefill(torch.tensor(t + [0] * (lim - len(t))), len(t))[0] for t in ids]
  waiting = list(range(len(ids)))
  owner: dict[int, int] = {}                 # slot -> prompt index
  out = [[] for _ in ids]
  eos = getattr(tok, "eos_id", None)
  while waiting or owner:
    for s in range(slots):
      if s not in owner and waiting:
        i = waiting.pop(0)
        state = eng.insert(prefixes[i], state, s)
        owner[s] = i
        out[i].append(int(prefixes[i].first_token))
    state, res = eng.generate(state)
    for s, i in list(owner.items()):
      t = int(res.data[s, 0])
      out[i].append(t)
      if len(out[i]) >= budget or (eos is not None and t == eos) or int(state.next_pos[s]) >= int(config.max_target_length) - 1:
        eng.free_slot(state, s)
        del owner[s]
  return [tok.decode(o) for o in out]


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  prompts = None
  rest = []
  for a in argv[1:]:
    if a.startswith("prompts="):
      prompts = a.split("=", 1)[1].split("|")
    else:
      rest.append(a)
  cfg = pyconfig.initialize([argv[0]] + rest)
  texts = decode_multi(cfg, prompts or [cfg.prompt])
  for p, t in zip(prompts or [cfg.prompt], texts):
    print(f"Input `{p}` -> `{t}`")
  return texts


if __name__ == "__main__":
  main()
