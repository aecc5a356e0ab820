"""Trains a SentencePiece vocabulary from the first characters of a text corpus.

  python -m maxtext.trainers.tokenizer.train_tokenizer --train_files='data/*.parquet' --file_type=parquet \
      --vocab_size=32768 --assets_path=assets --vocab_model_name=tokenizer

Same job as the reference's tool (src/maxtext/trainers/tokenizer/train_tokenizer.py:123-198): stream examples, dump up
to `max_corpus_chars` characters of the text column into a temporary file, run the SentencePiece trainer on it, and move
the model to `<assets_path>/<vocab_model_name>`. The reader is this package's file reader (jsonl, parquet, plain text;
`--grain_train_files` / `--grain_file_type` are accepted as aliases of `--train_files` / `--file_type`), and the
resulting model loads through `tokenizer_type=sentencepiece`.
"""
from __future__ import annotations

import argparse
import os
import shutil
import tempfile
import time

from ...input_pipeline.file_pipeline import _expand, _read_examples
from ...utils import max_logging


def example_texts(patterns: str, column: str = "text"):
  """Yields the text column of every example of the files matching `patterns`, files taken round-robin so that a prefix
  of the stream samples all of them."""
  files = _expand(patterns)
  if not files:
    raise FileNotFoundError(f"no files match {patterns!r}")
  readers = [_read_examples(f, column) for f in files]
  while readers:
    alive = []
    for r in readers:
      try:
        ex = next(r)
      except StopIteration:
        continue
      alive.append(r)
      val = ex.get(column) if isinstance(ex, dict) else ex
      if val is None:
        continue
      yield val.decode("utf-8") if isinstance(val, bytes) else str(val)
    readers = alive


def dump_chars_to_textfile(texts, max_chars: int) -> tuple[str, int]:
  """Writes texts, one per line, until `max_chars` characters were written; returns (path, characters written)."""
  count = 0
  with tempfile.NamedTemporaryFile(delete=False, prefix="ds_chars", mode="w", encoding="utf-8") as fh:
    for t in texts:
      line = t.replace("\n", " ") + "\n"
      fh.write(line)
      count += len(line)
      if count >= max_chars:
        break
  return fh.name, count


def train_sentencepiece(texts, *, vocab_size: int, model_path: str, max_chars: int = 10_000_000, model_type: str = "unigram",
                        character_coverage: float = 1.0) -> str:
  from sentencepiece import SentencePieceTrainer
  corpus, n = dump_chars_to_textfile(texts, max_chars)
  max_logging.log(f"tokenizer trainer: {n} characters dumped to {corpus}")
  with tempfile.TemporaryDirectory() as tmp:
    prefix = os.path.join(tmp, "sp")
    # ids match the reference's trainer: pad 0, eos 1, unk 2, no bos piece
    SentencePieceTrainer.Train(input=corpus, vocab_size=int(vocab_size), character_coverage=float(character_coverage), model_prefix=prefix,
                               model_type=model_type, pad_id=0, eos_id=1, unk_id=2, bos_id=-1, hard_vocab_limit=False,
                               input_sentence_size=0, shuffle_input_sentence=False, minloglevel=1)
    os.makedirs(os.path.dirname(os.path.abspath(model_path)), exist_ok=True)
    shutil.move(prefix + ".model", model_path)
  os.unlink(corpus)
  return model_path


def train_tokenizer(train_files: str, file_type: str = "parquet", data_column: str = "text", vocab_size: int = 32_768,
                    max_corpus_chars: int = 10_000_000, assets_path: str = "assets", vocab_model_name: str = "tokenizer") -> str:
  if file_type not in ("parquet", "jsonl", "json", "text", "txt"):
    raise ValueError(f"unsupported file type {file_type!r}: this reader covers parquet, jsonl and plain text")
  t0 = time.time()
  path = train_sentencepiece(example_texts(train_files, data_column), vocab_size=vocab_size, max_chars=max_corpus_chars,
                             model_path=os.path.join(assets_path, vocab_model_name))
  max_logging.log(f"tokenizer trainer: wrote {path} in {time.time() - t0:.1f} s")
  return path


def main(argv=None):
  ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
  ap.add_argument("--train_files", "--grain_train_files", dest="train_files", required=True)
  ap.add_argument("--file_type", "--grain_file_type", dest="file_type", default="parquet")
  ap.add_argument("--data_column", default="text")
  ap.add_argument("--vocab_size", type=int, default=32_768)
  ap.add_argument("--max_corpus_chars", type=int, default=10_000_000)
  ap.add_argument("--assets_path", default="assets")
  ap.add_argument("--vocab_model_name", default="tokenizer")
  a = ap.parse_args(argv)
  train_tokenizer(a.train_files, a.file_type, a.data_column, a.vocab_size, a.max_corpus_chars, a.assets_path, a.vocab_model_name)


if __name__ == "__main__":
  main()
