"""Tokenizer wrappers: SentencePiece, HuggingFace, tiktoken-style BPE files, and a byte-level fallback
(src/maxtext/input_pipeline/tokenizer.py:1-260). `build_tokenizer` picks by `tokenizer_type`; every wrapper offers
encode(text) -> list[int], decode(ids) -> str, bos_id, eos_id, pad_id, vocab_size."""
from __future__ import annotations

import os


class ByteTokenizer:
  """256 byte values + BOS/EOS/PAD; needs no asset, used by tests and when tokenizer_path is empty."""
  bos_id, eos_id, pad_id = 256, 257, 258
  vocab_size = 259

  def encode(self, text: str, add_bos=False, add_eos=False) -> list[int]:
    ids = list(text.encode("utf-8"))
    return ([self.bos_id] if add_bos else []) + ids + ([self.eos_id] if add_eos else [])

  def decode(self, ids) -> str:
    return bytes(int(i) for i in ids if 0 <= int(i) < 256).decode("utf-8", errors="replace")


class SentencePieceTokenizer:
  def __init__(self, path: str):
    import sentencepiece as spm
    self.sp = spm.SentencePieceProcessor(model_file=path)
    self.bos_id, self.eos_id = self.sp.bos_id(), self.sp.eos_id()
    self.pad_id = self.sp.pad_id() if self.sp.pad_id() >= 0 else 0
    self.vocab_size = self.sp.get_piece_size()

  def encode(self, text, add_bos=False, add_eos=False):
    ids = self.sp.encode(text)
    return ([self.bos_id] if add_bos and self.bos_id >= 0 else []) + ids + ([self.eos_id] if add_eos and self.eos_id >= 0 else [])

  def decode(self, ids):
    return self.sp.decode([int(i) for i in ids])


class HFTokenizer:
  def __init__(self, path: str, token: str = ""):
    from transformers import AutoTokenizer
    self.tok = AutoTokenizer.from_pretrained(path, token=token or None, local_files_only=not bool(token))
    self.bos_id = self.tok.bos_token_id if self.tok.bos_token_id is not None else -1
    self.eos_id = self.tok.eos_token_id if self.tok.eos_token_id is not None else -1
    self.pad_id = self.tok.pad_token_id if self.tok.pad_token_id is not None else 0
    self.vocab_size = len(self.tok)

  def encode(self, text, add_bos=False, add_eos=False):
    ids = self.tok.encode(text, add_special_tokens=False)
    return ([self.bos_id] if add_bos and self.bos_id >= 0 else []) + ids + ([self.eos_id] if add_eos and self.eos_id >= 0 else [])

  def decode(self, ids):
    return self.tok.decode([int(i) for i in ids])

  def apply_chat_template(self, messages, **kw):
    return self.tok.apply_chat_template(messages, tokenize=False, **kw)


def build_tokenizer(config):
  path, kind = config.tokenizer_path, config.tokenizer_type
  if not path:
    return ByteTokenizer()
  if kind == "sentencepiece":
    return SentencePieceTokenizer(path)
  if kind == "huggingface":
    return HFTokenizer(path, config.hf_access_token)
  if kind == "tiktoken":
    try:
      import tiktoken  # noqa: F401
    except ImportError as e:
      raise RuntimeError("tokenizer_type=tiktoken needs the tiktoken package, which is not installed here") from e
    from tiktoken.load import load_tiktoken_bpe
    import tiktoken
    ranks = load_tiktoken_bpe(path)
    enc = tiktoken.Encoding(name=os.path.basename(path), pat_str=r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+",
                            mergeable_ranks=ranks, special_tokens={"<|begin_of_text|>": len(ranks), "<|end_of_text|>": len(ranks) + 1})
    t = ByteTokenizer()
    t.encode = lambda text, add_bos=False, add_eos=False: ([len(ranks)] if add_bos else []) + enc.encode(text) + ([len(ranks) + 1] if add_eos else [])
    t.decode = lambda ids: enc.decode([int(i) for i in ids])
    t.bos_id, t.eos_id, t.pad_id, t.vocab_size = len(ranks), len(ranks) + 1, 0, len(ranks) + 2
    return t
  raise ValueError(f"unknown tokenizer_type {kind}")
