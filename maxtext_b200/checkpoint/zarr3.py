"""Minimal zarr v3 array reader/writer (numpy + stdlib only).

Orbax stores every leaf of a checkpoint pytree as a zarr array; with
`checkpoint_storage_use_ocdbt=False` (a legal mode of the reference, src/maxtext/configs/base.yml:75)
the arrays are plain directories `<leaf name>/zarr.json` + chunk files `c/<i>/<j>/...`. tensorstore and
orbax are not available here, so this module writes that layout directly: regular chunk grid,
little-endian `bytes` codec, no compression, bfloat16 stored as its 2-byte pattern with data_type
"bfloat16".
"""
from __future__ import annotations

import itertools
import json
import os

import numpy as np

try:
  import ml_dtypes
  _BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
  _BF16 = None

_NAMES = {"float32": np.float32, "float64": np.float64, "float16": np.float16, "int32": np.int32, "int64": np.int64,
          "int8": np.int8, "uint8": np.uint8, "bool": np.bool_, "uint32": np.uint32}


def _dtype_name(dt: np.dtype) -> str:
  if _BF16 is not None and dt == _BF16:
    return "bfloat16"
  return np.dtype(dt).name


def _dtype_of(name: str) -> np.dtype:
  if name == "bfloat16":
    return _BF16
  return np.dtype(_NAMES[name])


def write_meta(path: str, shape, chunks, dtype: np.dtype):
  os.makedirs(path, exist_ok=True)
  meta = {
      "zarr_format": 3, "node_type": "array", "shape": list(shape), "data_type": _dtype_name(dtype),
      "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": list(chunks)}},
      "chunk_key_encoding": {"name": "default", "configuration": {"separator": "/"}},
      "fill_value": 0, "codecs": [{"name": "bytes", "configuration": {"endian": "little"}}],
      "attributes": {}, "dimension_names": None,
  }
  with open(os.path.join(path, "zarr.json"), "w", encoding="utf-8") as fh:
    json.dump(meta, fh)


def chunk_path(path: str, index) -> str:
  return os.path.join(path, "c", *[str(i) for i in index]) if len(index) else os.path.join(path, "c")


def write_chunk(path: str, index, data: np.ndarray):
  p = chunk_path(path, index)
  os.makedirs(os.path.dirname(p), exist_ok=True)
  tmp = f"{p}.tmp{os.getpid()}"           # unique per writer: a stray second writer must not break the rename
  with open(tmp, "wb") as fh:
    fh.write(np.ascontiguousarray(data).tobytes())
  os.replace(tmp, p)


def write_array(path: str, arr: np.ndarray, chunks=None):
  chunks = tuple(chunks) if chunks is not None else tuple(arr.shape)
  write_meta(path, arr.shape, chunks, arr.dtype)
  if arr.ndim == 0:
    write_chunk(path, (), arr)
    return
  grid = [range(-(-s // c)) for s, c in zip(arr.shape, chunks)]
  for idx in itertools.product(*grid):
    sl = tuple(slice(i * c, min((i + 1) * c, s)) for i, c, s in zip(idx, chunks, arr.shape))
    block = arr[sl]
    if block.shape != chunks:
      full = np.zeros(chunks, dtype=arr.dtype)
      full[tuple(slice(0, n) for n in block.shape)] = block
      block = full
    write_chunk(path, idx, block)


def read_meta(path: str) -> dict:
  with open(os.path.join(path, "zarr.json"), "r", encoding="utf-8") as fh:
    return json.load(fh)


def read_array(path: str, region=None) -> np.ndarray:
  """Read the whole array, or the hyper-rectangle `region` (tuple of slices) touching only its chunks."""
  meta = read_meta(path)
  shape = tuple(meta["shape"])
  chunks = tuple(meta["chunk_grid"]["configuration"]["chunk_shape"])
  dt = _dtype_of(meta["data_type"])
  if len(shape) == 0:
    return np.frombuffer(open(chunk_path(path, ()), "rb").read(), dtype=dt).reshape(())
  region = tuple(region) if region is not None else tuple(slice(0, s) for s in shape)
  region = tuple(slice(*r.indices(s)) for r, s in zip(region, shape))
  out = np.zeros(tuple(r.stop - r.start for r in region), dtype=dt)
  grid = [range(r.start // c, -(-r.stop // c)) for r, c in zip(region, chunks)]
  for idx in itertools.product(*grid):
    p = chunk_path(path, idx)
    if not os.path.exists(p):
      continue
    block = np.frombuffer(open(p, "rb").read(), dtype=dt).reshape(chunks)
    src, dst = [], []
    for i, c, r in zip(idx, chunks, region):
      lo, hi = max(r.start, i * c), min(r.stop, (i + 1) * c)
      src.append(slice(lo - i * c, hi - i * c))
      dst.append(slice(lo - r.start, hi - r.start))
    out[tuple(dst)] = block[tuple(src)]
  return out
