"""Tensor-parallel all-reduce fused with the GEMM that produces its input.

A row-parallel linear (attention output, MLP down projection) yields partial sums that must be added over the tensor-parallel
ranks; so does the input gradient of a column-parallel linear. The reference leaves both to XLA's all-reduce /
collective-matmul passes. Here the GEMM kernel's epilogue adds every finished output tile straight
into the fp32 accumulation buffer of the rank that owns those rows (a TMA reduce-add into peer memory over NVLink, tile by
tile while later tiles are still being computed), and one more kernel reads the owners' reduced chunks back, converting to
bf16 (the all-gather half). Epoch-flag barriers separate the phases; see TPReduceRuntime for the two variants (staged
stores, the default, and fp32 reduce-adds).
"""
from __future__ import annotations

import torch

from ..ops import backend
from . import symm as symm_lib

_RT: dict = {}


class TPReduceRuntime:
  """mode "staged" (default): partial tiles are STORED as bf16 into the owner's staging slot for the source rank, the owner
  sums the staged copies in rank order (bitwise reproducible, same bytes over NVLink as a bf16 all-reduce), peers pull the
  reduced chunks. mode "atomic": tiles are ADDED in fp32 into the owner's accumulator by TMA reduce-add (more exact, twice
  the bytes, and remote reductions are slow beyond two ranks: 4.1 ms vs 1.4 ms for GEMM + NCCL at eight ranks)."""

  def __init__(self, group, device, rows: int, n: int, mode: str = "staged"):
    self.symm = symm_lib.SymmGroup(group, device)
    self.world, self.rank = self.symm.world, self.symm.rank
    assert rows % (self.world * 128) == 0 and n % 128 == 0
    self.rows, self.n, self.mode = rows, n, mode
    self.chunk_rows = rows // self.world
    self.chunk = self.chunk_rows * n
    E = backend.ext()
    dev = torch.device(device)
    if mode == "atomic":
      self.acc, self.maps = [], []
      for _ in range(3):
        b = self.symm.alloc(self.chunk, torch.float32, zero=True)
        self.acc.append(b)
        self.maps.append(E.gemm_rs_maps(b.ptrs, self.chunk_rows, n, dev, False))
    else:
      self.staging = self.symm.alloc(self.world * self.chunk, torch.bfloat16)       # [source rank][chunk]
      self.reduced = self.symm.alloc(self.chunk, torch.bfloat16)
      mine = [p + self.rank * self.chunk * 2 for p in self.staging.ptrs]            # my slot inside every owner's staging area
      self.maps = E.gemm_rs_maps(mine, self.chunk_rows, n, dev, True)
    self.use = 0
    self.symm.barrier(1)
    torch.cuda.synchronize(device)

  def all_reduce_gemm(self, a: torch.Tensor, w: torch.Tensor, tb: bool) -> torch.Tensor:
    """sum over ranks of a @ (w.T if tb else w); a [rows, k_local] bf16; returns [rows, n] bf16 on every rank."""
    E = backend.ext()
    out = torch.empty(self.rows, self.n, dtype=torch.bfloat16, device=a.device)
    if self.mode == "atomic":
      i, nxt = self.use % 3, (self.use + 1) % 3
      self.use += 1
      self.acc[nxt].tensor.zero_()
      E.gemm_rs(a, w, tb, self.maps[i], self.world, False)
      self.symm.signal(2)
      self.symm.wait(2)
      E.gather_cvt(self.acc[i].table, self.chunk, self.world, out)
      return out
    self.use += 1
    E.gemm_rs(a, w, tb, self.maps, self.world, True)          # epilogue stores every tile into its owner's staging slot
    self.symm.signal(2)
    self.symm.wait(2)                                         # all partials of my rows have landed
    E.reduce_staged(self.staging.tensor, self.world, self.reduced.tensor)
    self.symm.signal(3)
    self.symm.wait(3)                                         # every owner's reduced chunk is ready (and my staging area is free again)
    E.gather_segments(self.reduced.table, out, self.chunk * 2, 256 * 1024, self.world, 296)
    return out


def runtime_for(ctx, x: torch.Tensor, n: int):
  """The fused all-reduce runtime for activations shaped like `x` (rows = all leading dims), or None if not applicable."""
  c = ctx.config
  if ctx.tp_size <= 1 or getattr(ctx, "sp", False) or not x.is_cuda or x.dtype != torch.bfloat16 or not bool(getattr(c, "use_fused_comm_kernels", False)):
    return None
  rows = x.numel() // x.shape[-1]
  if ctx.tp_size > int(getattr(c, "tp_fused_max_ranks", 2)):
    return None        # measured: faster than GEMM + NCCL at 2 ranks (1.16x), slower at 8 where NCCL reduces inside the switch
  if rows % (ctx.tp_size * 128) or n % 128 or not symm_lib.available() or not hasattr(backend.ext(), "gemm_rs"):
    return None
  key = (id(ctx.tp_group), rows, n)
  if key not in _RT:
    _RT[key] = TPReduceRuntime(ctx.tp_group, x.device, rows, n)
  return _RT[key]
