"""Tensor-parallel all-reduce fused with the GEMM that produces its input.

A row-parallel linear (attention output, MLP down projection) yields partial sums that must be added over the tensor-parallel
ranks; so does the input gradient of a column-parallel linear. The reference leaves both to XLA's all-reduce /
collective-matmul passes ("TP"). Here the GEMM kernel's epilogue adds every finished output tile straight
into the fp32 accumulation buffer of the rank that owns those rows (a TMA reduce-add into peer memory over NVLink, tile by
tile while later tiles are still being computed), and one more kernel reads the owners' reduced chunks back, converting to
bf16 (the all-gather half). One epoch-flag barrier separates the two.

Three accumulation buffers rotate: use i adds into buffer i % 3 while buffer (i + 1) % 3 is being zeroed for the next use;
readers of a buffer's previous use are known to be done because they signalled the flag of the use in between.
Sums of more than two ranks depend on arrival order in the last bit (fp32); two ranks are bitwise reproducible.
"""
from __future__ import annotations

import torch

from ..ops import backend
from . import symm as symm_lib

_RT: dict = {}


class TPReduceRuntime:
  def __init__(self, group, device, rows: int, n: int):
    self.symm = symm_lib.SymmGroup(group, device)
    self.world, self.rank = self.symm.world, self.symm.rank
    assert rows % (self.world * 128) == 0 and n % 128 == 0
    self.rows, self.n = rows, n
    self.chunk_rows = rows // self.world
    E = backend.ext()
    self.acc, self.maps = [], []
    for _ in range(3):
      b = self.symm.alloc(self.chunk_rows * n, torch.float32, zero=True)
      self.acc.append(b)
      self.maps.append(E.gemm_rs_maps(b.ptrs, self.chunk_rows, n, torch.device(device)))
    self.use = 0
    self.symm.barrier(1)
    torch.cuda.synchronize(device)

  def all_reduce_gemm(self, a: torch.Tensor, w: torch.Tensor, tb: bool) -> torch.Tensor:
    """sum over ranks of a @ (w.T if tb else w); a [rows, k_local] bf16; returns [rows, n] bf16 on every rank."""
    E = backend.ext()
    i, nxt = self.use % 3, (self.use + 1) % 3
    self.use += 1
    self.acc[nxt].tensor.zero_()
    E.gemm_rs(a, w, tb, self.maps[i], self.world)
    self.symm.signal(2)
    self.symm.wait(2)
    out = torch.empty(self.rows, self.n, dtype=torch.bfloat16, device=a.device)
    E.gather_cvt(self.acc[i].table, self.chunk_rows * self.n, self.world, out)
    return out


def runtime_for(ctx, x: torch.Tensor, n: int):
  """The fused all-reduce runtime for activations shaped like `x` (rows = all leading dims), or None if not applicable."""
  c = ctx.config
  if ctx.tp_size <= 1 or not x.is_cuda or x.dtype != torch.bfloat16 or not bool(getattr(c, "use_fused_comm_kernels", False)):
    return None
  rows = x.numel() // x.shape[-1]
  if rows % (ctx.tp_size * 128) or n % 128 or not symm_lib.available() or not hasattr(backend.ext(), "gemm_rs"):
    return None
  key = (id(ctx.tp_group), rows, n)
  if key not in _RT:
    _RT[key] = TPReduceRuntime(ctx.tp_group, x.device, rows, n)
  return _RT[key]
