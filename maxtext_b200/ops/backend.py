"""Loader for the compiled sm_100a kernel library.

The extension is built in-tree by `maxtext_b200.csrc.build` (one shared object,
`csrc/build/maxtext_b200_C.so`). On a machine with a CUDA device the library is mandatory: a
missing or unloadable build raises instead of silently running PyTorch ops. On CPU-only machines
`ext()` returns None and callers use the PyTorch reference implementations.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import torch

_EXT = None
_TRIED = False
EXT_NAME = "maxtext_b200_C"
BUILD_DIR = os.path.normpath(os.path.join(os.path.dirname(__file__), "..", "csrc", "build"))


def so_path() -> str:
  return os.path.join(BUILD_DIR, EXT_NAME + ".so")


def _import_so(path: str):
  spec = importlib.util.spec_from_file_location(EXT_NAME, path)
  mod = importlib.util.module_from_spec(spec)
  spec.loader.exec_module(mod)
  sys.modules[EXT_NAME] = mod
  return mod


def ext(required: bool | None = None):
  """Return the extension module (cached). `required` defaults to "a CUDA device is present"."""
  global _EXT, _TRIED
  if _EXT is not None:
    return _EXT
  if required is None:
    required = torch.cuda.is_available()
  if _TRIED and not required:
    return None
  _TRIED = True
  path = so_path()
  err = None
  if os.path.isfile(path):
    try:
      _EXT = _import_so(path)
      return _EXT
    except Exception as e:  # pylint: disable=broad-except
      err = e
  if required:
    if os.environ.get("MAXTEXT_B200_JIT_BUILD", "1") == "1" and err is None:
      from ..csrc import build as _build
      _build.build_extension(verbose=False)
      _EXT = _import_so(path)
      return _EXT
    raise RuntimeError(
        f"maxtext_b200: CUDA kernel library {path} is missing or failed to load ({err}); "
        "run `python -c 'import __graft_entry__ as g; g.build()'` first. Refusing to fall back to PyTorch ops on a GPU.")
  return None


def have_ext() -> bool:
  try:
    return ext(required=False) is not None
  except Exception:  # pylint: disable=broad-except
    return False


def use_cuda_kernels(t: torch.Tensor) -> bool:
  """True when `t` lives on a GPU (then the extension must be present)."""
  if not t.is_cuda:
    return False
  ext(required=True)
  return True
