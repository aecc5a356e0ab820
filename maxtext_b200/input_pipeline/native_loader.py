"""Iterator over pre-tokenized files backed by the native loader (`csrc/host/data_loader.cpp`).

`dataset_type=tokens` (or any file pipeline pointed at `.bin` / `.npy` int32 token files with `use_native_loader=true`)
uses it: a C++ thread memory-maps the files, packs documents into rows and keeps a few batches ready, and `__next__`
copies one into reusable pinned tensors. Its state (file, offset, document, epoch) goes into checkpoints through the
same `state()` / `load_state()` hooks as the Python pipelines, so a resumed run continues with the next batch."""
from __future__ import annotations

import importlib.util
import os

import torch

_HOST = None


def host_lib(build: bool = True):
  """The host runtime library; built in-tree on first use when it is not there yet."""
  global _HOST
  if _HOST is not None:
    return _HOST
  here = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
  so = os.path.join(here, "build_host", "maxtext_b200_host.so")
  if not os.path.isfile(so):
    if not build:
      return None
    from ..csrc import build as b
    b.build_host_extension(verbose=False)
  spec = importlib.util.spec_from_file_location("maxtext_b200_host", so)
  mod = importlib.util.module_from_spec(spec)
  spec.loader.exec_module(mod)
  _HOST = mod
  return mod


class NativeTokenIterator:
  def __init__(self, files: list[str], seq_len: int, batch_size: int, eos_id: int, data_rank: int = 0, data_world: int = 1,
               prefetch: int = 4, pin: bool | None = None):
    self.files, self.seq, self.batch = list(files), int(seq_len), int(batch_size)
    self._loader = host_lib().TokenLoader(self.files, self.seq, self.batch, int(eos_id), int(data_rank), int(data_world), int(prefetch))
    pin = torch.cuda.is_available() if pin is None else pin
    mk = lambda: torch.empty(self.batch, self.seq, dtype=torch.int32, pin_memory=pin)  # noqa: E731
    # two sets of host buffers: the one handed out last may still be the source of an asynchronous copy to the device
    self._bufs = [tuple(mk() for _ in range(4)) for _ in range(2)]
    self._flip = 0

  def __iter__(self):
    return self

  def __next__(self) -> dict:
    inp, tgt, seg, pos = self._bufs[self._flip]
    self._flip ^= 1
    self._loader.next(inp, tgt, seg, pos)
    return {"inputs": inp, "targets": tgt, "inputs_segmentation": seg, "targets_segmentation": seg, "inputs_position": pos}

  def state(self) -> dict:
    return {"native_position": [int(v) for v in self._loader.state()]}

  def load_state(self, st: dict):
    if st and "native_position" in st:
      self._loader.seek([int(v) for v in st["native_position"]])
