"""Record containers that the reference reads through TFDS / Grain (src/maxtext/input_pipeline/tfds_data_processing.py,
grain_data_processing.py), decoded here without TensorFlow:

  * TFRecord files: [u64 length][u32 masked crc32c(length)][payload][u32 masked crc32c(payload)] per record;
  * `tf.train.Example` payloads: the protobuf wire format of Example -> Features -> map<string, Feature>, where a Feature is
    a bytes / float / int64 list;
  * Arrow IPC files and streams (what `datasets.save_to_disk` and the HF cache write), through pyarrow.

A writer for the first two exists for tests and for converting small corpora.
"""
from __future__ import annotations

import struct

import numpy as np

# ------------------------------------------------------------------------------------------------- crc32c (Castagnoli)
_TABLE = None


def _table():
  global _TABLE
  if _TABLE is None:
    t = np.zeros(256, dtype=np.uint32)
    for i in range(256):
      c = i
      for _ in range(8):
        c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1
      t[i] = c
    _TABLE = t.tolist()
  return _TABLE


def crc32c(data: bytes) -> int:
  t = _table()
  c = 0xFFFFFFFF
  for b in data:
    c = t[(c ^ b) & 0xFF] ^ (c >> 8)
  return c ^ 0xFFFFFFFF


def masked_crc(data: bytes) -> int:
  c = crc32c(data)
  return ((((c >> 15) | (c << 17)) & 0xFFFFFFFF) + 0xA282EAD8) & 0xFFFFFFFF


# ------------------------------------------------------------------------------------------------- TFRecord
def read_tfrecord(path: str, verify_payload: bool = False):
  """Yields the raw payload of every record. The length checksum is always verified (it guards the framing); the payload
  checksum only on request (a byte loop in Python)."""
  with open(path, "rb") as fh:
    while True:
      head = fh.read(12)
      if not head:
        return
      if len(head) < 12:
        raise IOError(f"{path}: truncated record header")
      (n,), (crc,) = struct.unpack("<Q", head[:8]), struct.unpack("<I", head[8:])
      if masked_crc(head[:8]) != crc:
        raise IOError(f"{path}: corrupt record length")
      data = fh.read(n)
      tail = fh.read(4)
      if len(data) < n or len(tail) < 4:
        raise IOError(f"{path}: truncated record")
      if verify_payload and masked_crc(data) != struct.unpack("<I", tail)[0]:
        raise IOError(f"{path}: corrupt record payload")
      yield data


def write_tfrecord(path: str, payloads):
  with open(path, "wb") as fh:
    for data in payloads:
      head = struct.pack("<Q", len(data))
      fh.write(head + struct.pack("<I", masked_crc(head)) + data + struct.pack("<I", masked_crc(data)))


# ------------------------------------------------------------------------------------------------- tf.train.Example
def _varint(buf, i):
  shift = val = 0
  while True:
    b = buf[i]
    i += 1
    val |= (b & 0x7F) << shift
    if not b & 0x80:
      return val, i
    shift += 7


def _fields(buf):
  """(field number, wire type, value) of one message; value is int for varints / fixed, memoryview for length-delimited."""
  i, n = 0, len(buf)
  while i < n:
    key, i = _varint(buf, i)
    num, wt = key >> 3, key & 7
    if wt == 0:
      v, i = _varint(buf, i)
    elif wt == 1:
      v, i = bytes(buf[i:i + 8]), i + 8
    elif wt == 2:
      ln, i = _varint(buf, i)
      v, i = buf[i:i + ln], i + ln
    elif wt == 5:
      v, i = bytes(buf[i:i + 4]), i + 4
    else:
      raise ValueError(f"unsupported protobuf wire type {wt}")
    yield num, wt, v


def _feature(buf):
  for num, _, v in _fields(buf):
    if num == 1:                                                   # BytesList
      return [bytes(x) for n_, _, x in _fields(v) if n_ == 1]
    if num == 2:                                                   # FloatList (packed or not)
      out = []
      for n_, wt, x in _fields(v):
        if n_ == 1:
          out.extend(np.frombuffer(bytes(x), dtype="<f4").tolist() if wt == 2 else [struct.unpack("<f", x)[0]])
      return np.asarray(out, dtype=np.float32)
    if num == 3:                                                   # Int64List (packed or not)
      out = []
      for n_, wt, x in _fields(v):
        if n_ != 1:
          continue
        if wt == 2:
          j = 0
          while j < len(x):
            val, j = _varint(x, j)
            out.append(val - (1 << 64) if val >> 63 else val)
        else:
          out.append(x - (1 << 64) if x >> 63 else x)
      return np.asarray(out, dtype=np.int64)
  return []


def parse_example(payload: bytes) -> dict:
  """Serialized tf.train.Example -> {name: [bytes, ...] | float32 array | int64 array}."""
  buf = memoryview(payload)
  out = {}
  for num, _, feats in _fields(buf):
    if num != 1:
      continue
    for n2, _, entry in _fields(feats):                           # map entries: key = 1, value = 2
      if n2 != 1:
        continue
      key, val = None, []
      for n3, _, x in _fields(entry):
        if n3 == 1:
          key = bytes(x).decode("utf-8")
        elif n3 == 2:
          val = _feature(x)
      if key is not None:
        out[key] = val
  return out


def _enc_varint(v: int) -> bytes:
  v &= (1 << 64) - 1
  out = bytearray()
  while True:
    b = v & 0x7F
    v >>= 7
    out.append(b | (0x80 if v else 0))
    if not v:
      return bytes(out)


def _ld(num: int, data: bytes) -> bytes:
  return _enc_varint((num << 3) | 2) + _enc_varint(len(data)) + data


def build_example(features: dict) -> bytes:
  """{name: str | bytes | list of ints | list of floats} -> serialized tf.train.Example."""
  entries = b""
  for k, v in features.items():
    if isinstance(v, (str, bytes)):
      v = [v]
    v = list(v)
    if v and isinstance(v[0], (str, bytes)):
      body = _ld(1, b"".join(_ld(1, x.encode("utf-8") if isinstance(x, str) else x) for x in v))
    elif v and isinstance(v[0], float):
      body = _ld(2, _ld(1, np.asarray(v, dtype="<f4").tobytes()))
    else:
      body = _ld(3, _ld(1, b"".join(_enc_varint(int(x)) for x in v)))
    entries += _ld(1, _ld(1, k.encode("utf-8")) + _ld(2, body))
  return _ld(1, entries)


def read_tfrecord_examples(path: str, text_columns=()):
  """Examples of a TFRecord file as dicts; byte features named in `text_columns` (or all single-valued ones) become str."""
  for payload in read_tfrecord(path):
    ex = parse_example(payload)
    row = {}
    for k, v in ex.items():
      if isinstance(v, list) and v and isinstance(v[0], bytes):
        if len(v) == 1 and (not text_columns or k in text_columns):
          row[k] = v[0].decode("utf-8", errors="replace")
        else:
          row[k] = v
      else:
        row[k] = v
    yield row


# ------------------------------------------------------------------------------------------------- Arrow IPC
def read_arrow(path: str):
  """Rows of an Arrow IPC file or stream (HF `datasets` on-disk format), one record batch at a time."""
  import pyarrow as pa
  with pa.memory_map(path, "r") as src:
    try:
      reader = pa.ipc.open_stream(src)
      batches = iter(reader)
    except pa.ArrowInvalid:
      src.seek(0)
      reader = pa.ipc.open_file(src)
      batches = (reader.get_batch(i) for i in range(reader.num_record_batches))
    for batch in batches:
      yield from batch.to_pylist()
