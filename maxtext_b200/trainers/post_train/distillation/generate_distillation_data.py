"""Response-based distillation data: run a teacher over a prompt set and keep its answers as a fine-tuning set
(tools/data_generation/generate_distillation_data.py).

  python -m maxtext_b200.trainers.post_train.distillation.generate_distillation_data <teacher.yml> [key=value ...] \\
      --dataset prompts.jsonl [--column messages|prompt] --out distill.jsonl [--num-generations 2] [--batch-size 64] [--num-batches N] \\
      [--max-new-tokens 256] [--use-chat-template]

Input rows are JSON lines (or parquet) with either a `messages` list (the conversation up to the point where the teacher
should answer; a trailing assistant turn is dropped) or a plain `prompt`. Prompts longer than `max_prefill_predict_length`
tokens are skipped, as the reference does. Every kept prompt gets `--num-generations` answers (sampling per
`decode_sampling_strategy`), written as `{"prompt": ..., "completion": ..., "messages": [... + assistant]}` rows that the SFT
pipeline reads directly. The teacher runs in-process on the decode engine (slot batching); `--server URL` sends the prompts to a
running `maxengine_server` instead.
"""
from __future__ import annotations

import argparse
import json
import sys


def read_rows(path: str) -> list[dict]:
  if path.endswith(".parquet"):
    import pyarrow.parquet as pq
    return pq.read_table(path).to_pylist()
  with open(path, encoding="utf-8") as fh:
    return [json.loads(line) for line in fh if line.strip()]


def prompt_of(row: dict, column: str, template: str | None):
  """(prompt text, messages without the final assistant turn or None)."""
  v = row.get(column)
  if isinstance(v, list):
    msgs = list(v)
    while msgs and msgs[-1].get("role") == "assistant":
      msgs.pop()
    if not msgs:
      return None, None
    from ....input_pipeline import chat
    return chat.render(msgs, template or chat.DEFAULT_TEMPLATE, add_generation_prompt=True), msgs
  if v is None:
    return None, None
  text = str(v)
  if template:
    from ....input_pipeline import chat
    msgs = [{"role": "user", "content": text}]
    return chat.render(msgs, template, add_generation_prompt=True), msgs
  return text, None


def generate(rows, generate_fn, count_tokens, max_prompt_tokens: int, column: str = "messages", template: str | None = None,
             num_generations: int = 1, batch_size: int = 64, num_batches: int | None = None, max_new_tokens: int = 256):
  """Yields output rows. `generate_fn(list of prompts, max_new_tokens) -> list of texts`; `count_tokens(text) -> int`."""
  kept, skipped = [], 0
  for row in rows:
    text, msgs = prompt_of(row, column, template)
    if text is None or count_tokens(text) > max_prompt_tokens:
      skipped += 1
      continue
    kept.append((text, msgs))
  if num_batches is not None:
    kept = kept[: num_batches * batch_size]
  for b0 in range(0, len(kept), batch_size):
    chunk = kept[b0:b0 + batch_size]
    for g in range(num_generations):
      outs = generate_fn([t for t, _ in chunk], max_new_tokens)
      for (text, msgs), completion in zip(chunk, outs):
        row = {"prompt": text, "completion": completion, "generation": g}
        if msgs is not None:
          row["messages"] = msgs + [{"role": "assistant", "content": completion}]
        yield row
  generate.skipped = skipped


def main(argv=None):
  argv = list(sys.argv[1:] if argv is None else argv)
  ap = argparse.ArgumentParser()
  ap.add_argument("config", nargs="+")
  ap.add_argument("--dataset", required=True)
  ap.add_argument("--column", default="messages")
  ap.add_argument("--out", required=True)
  ap.add_argument("--num-generations", type=int, default=1)
  ap.add_argument("--batch-size", type=int, default=64)
  ap.add_argument("--num-batches", type=int)
  ap.add_argument("--max-new-tokens", type=int, default=256)
  ap.add_argument("--use-chat-template", action="store_true")
  ap.add_argument("--server", default="")
  a = ap.parse_args(argv)
  from ....config import pyconfig
  from ....eval.runner import LocalBackend, ServerBackend
  from ....input_pipeline import chat
  cfg = pyconfig.initialize(["distill"] + a.config)
  backend = ServerBackend(a.server) if a.server else LocalBackend(cfg, slots=max(1, int(cfg.per_device_batch_size)))
  from ....input_pipeline.tokenizer import build_tokenizer
  tok = build_tokenizer(cfg)
  template = chat.load_template(cfg) if a.use_chat_template else None
  n = 0
  with open(a.out, "w", encoding="utf-8") as fh:
    for row in generate(read_rows(a.dataset), backend.generate, lambda t: len(tok.encode(t)), int(cfg.max_prefill_predict_length), a.column,
                        template, a.num_generations, a.batch_size, a.num_batches, a.max_new_tokens):
      fh.write(json.dumps(row) + "\n")
      n += 1
  print(json.dumps({"written": n, "skipped_prompts": getattr(generate, "skipped", 0), "out": a.out}))
  return n


if __name__ == "__main__":
  main()
