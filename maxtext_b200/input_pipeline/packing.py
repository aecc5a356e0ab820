"""Sequence packing with segment ids and per-segment positions
(src/maxtext/input_pipeline/packing/sequence_packing.py): first-fit, best-fit and concat-then-split."""
from __future__ import annotations

import numpy as np


def pack_first_fit(examples, seq_len: int, max_segments: int = -1, mode: str = "first_fit"):
  """examples: iterable of 1-D int arrays (already truncated to seq_len). Yields dict rows of length seq_len with
  tokens, segment ids (1-based, 0 = padding) and positions restarting at 0 in every segment."""
  bins: list[list[np.ndarray]] = []
  space: list[int] = []
  for ex in examples:
    ex = np.asarray(ex)[:seq_len]
    n = len(ex)
    if n == 0:
      continue
    cand = [i for i, s in enumerate(space) if s >= n and (max_segments <= 0 or len(bins[i]) < max_segments)]
    if cand:
      i = cand[0] if mode == "first_fit" else min(cand, key=lambda j: space[j] - n)
      bins[i].append(ex)
      space[i] -= n
    else:
      bins.append([ex])
      space.append(seq_len - n)
  for b in bins:
    yield _emit(b, seq_len)


def _emit(parts, seq_len):
  tok = np.zeros(seq_len, dtype=np.int32)
  seg = np.zeros(seq_len, dtype=np.int32)
  pos = np.zeros(seq_len, dtype=np.int32)
  o = 0
  for i, p in enumerate(parts):
    n = len(p)
    tok[o:o + n], seg[o:o + n], pos[o:o + n] = p, i + 1, np.arange(n)
    o += n
  return {"tokens": tok, "segmentation": seg, "position": pos}


def concat_then_split(examples, seq_len: int):
  """Concatenate everything and cut rows of seq_len; segment ids still mark document boundaries."""
  buf_t, buf_s, buf_p, sid = [], [], [], 1
  for ex in examples:
    ex = np.asarray(ex)
    buf_t.extend(ex.tolist())
    buf_s.extend([sid] * len(ex))
    buf_p.extend(range(len(ex)))
    sid += 1
    while len(buf_t) >= seq_len:
      s = np.asarray(buf_s[:seq_len])
      yield {"tokens": np.asarray(buf_t[:seq_len], dtype=np.int32), "segmentation": (s - s.min() + 1).astype(np.int32),
             "position": np.asarray(buf_p[:seq_len], dtype=np.int32)}
      buf_t, buf_s, buf_p = buf_t[seq_len:], buf_s[seq_len:], buf_p[seq_len:]


def shift_for_lm(row: dict, seq_len_plus_1: bool = True) -> dict:
  """tokens of length S+1 -> inputs/targets of length S with matching segmentation and positions; a target is
  masked (segmentation 0) where it crosses into another segment or padding."""
  t, s, p = row["tokens"], row["segmentation"], row["position"]
  tgt_seg = np.where(s[1:] == s[:-1], s[1:], 0)
  if (t < 0).any():
    # supervised fine-tuning on completions only: prompt tokens travel through packing as -(id + 1) and are never targets
    prompt = t < 0
    t = np.where(prompt, -t - 1, t).astype(np.int32)
    tgt_seg = np.where(prompt[1:], 0, tgt_seg)
  return {"inputs": t[:-1], "targets": t[1:], "inputs_segmentation": s[:-1], "targets_segmentation": tgt_seg.astype(np.int32),
          "inputs_position": p[:-1], "targets_position": p[:-1]}
