"""Symmetric memory over NVLink: buffers that every rank of a node can address, plus epoch flags.

MaxText has no communication code of its own: XLA lowers collectives to NCCL. Here, next to the
NCCL process groups of `parallel.mesh`, each shard group owns a *symmetric heap*: every rank allocates the same
buffers and exchanges handles, so a kernel running on one GPU can load from (or store to) the same offset of a
peer's buffer with plain memory instructions. The fused kernels of `csrc/comm_sm100.cu` and the all-gather GEMM
of `csrc/gemm_sm100.cu` take tables of such peer pointers.

Allocation and handle exchange use `torch.distributed._symmetric_memory` (CUDA VMM + fd passing under the hood);
everything that moves data is this repository's kernels. Synchronisation is by monotonically increasing epochs:
`signal(slot)` writes this rank's epoch into every peer's flag row, `wait(slot)` spins on the local row until all
peers reached it, with a time limit after which the kernel records a status code and returns (the host raises
`CommTimeoutError` when it next checks `kernel_status`).
"""
from __future__ import annotations

import os
import weakref

import torch
import torch.distributed as dist

from ..ops import backend


class CommTimeoutError(RuntimeError):
  pass


def available() -> bool:
  if not torch.cuda.is_available():
    return False
  try:
    import torch.distributed._symmetric_memory as sm  # noqa: F401
    return True
  except Exception:  # pylint: disable=broad-except
    return False


class SymmTensor:
  """A local tensor plus the device addresses of the same allocation on every rank of the group."""

  def __init__(self, tensor: torch.Tensor, ptrs: list[int], mc_ptr: int = 0):
    self.tensor = tensor
    self.ptrs = list(ptrs)
    self.mc_ptr = int(mc_ptr)          # multicast (NVLS) address of the allocation, 0 when the platform has none
    self.table = torch.tensor(self.ptrs, dtype=torch.int64, device=tensor.device)

  def table_at(self, elem_offset: int) -> torch.Tensor:
    """Pointer table of the sub-buffer that starts `elem_offset` elements into the allocation."""
    if elem_offset == 0:
      return self.table
    return self.table + elem_offset * self.tensor.element_size()


_LIVE: "weakref.WeakSet" = weakref.WeakSet()


def verify_all_canaries() -> int:
  """Checks the guard pages of every live group (no-op unless MAXTEXT_B200_CANARIES=1); returns how many buffers were checked."""
  n = 0
  for g in list(_LIVE):
    if g.canaries:
      g.verify_canaries()
      n += len(g._guards)
  return n


class SymmGroup:
  N_SLOTS = 16

  def __init__(self, group, device, wait_limit_ms: float | None = None):
    import torch.distributed._symmetric_memory as sm
    self._sm = sm
    self.group = group if group is not None else dist.group.WORLD
    self.device = torch.device(device)
    self.rank = dist.get_rank(self.group)
    self.world = dist.get_world_size(self.group)
    # how long a device-side flag wait may spin before it records a status code and returns (MAXTEXT_B200_WAIT_LIMIT_MS overrides:
    # tests use a few seconds so that a rank that lost its peer leaves on its own instead of being killed)
    self.wait_limit_ms = float(wait_limit_ms if wait_limit_ms is not None else os.environ.get("MAXTEXT_B200_WAIT_LIMIT_MS", 20000.0))
    self._handles = []
    # MAXTEXT_B200_CANARIES=1 (tests): every allocation is framed by two guard pages holding a fixed pattern; `check()` verifies
    # them, so a kernel (this rank's or a peer's) that wrote outside a symmetric buffer is caught at the next check
    self.canaries = os.environ.get("MAXTEXT_B200_CANARIES") == "1"
    self._guards: list[tuple[torch.Tensor, torch.Tensor]] = []
    self.flags = self.alloc(self.N_SLOTS * self.world, torch.int32, zero=True)
    self.epochs = [0] * self.N_SLOTS
    _LIVE.add(self)
    dist.barrier(group=self.group)

  GUARD_BYTES = 4096
  GUARD_WORD = 0x5AC3A55A

  def alloc(self, numel: int, dtype: torch.dtype, zero: bool = False) -> SymmTensor:
    guard = self.GUARD_BYTES // torch.empty((), dtype=dtype).element_size() if self.canaries else 0
    t = self._sm.empty(int(numel) + 2 * guard, dtype=dtype, device=self.device)
    if zero:
      t.zero_()
      torch.cuda.synchronize(self.device)
    hdl = self._sm.rendezvous(t, self.group.group_name if hasattr(self.group, "group_name") else self.group)
    self._handles.append(hdl)
    ptrs = [int(p) for p in hdl.buffer_ptrs]
    # torch hands out one slab per rendezvous; the tensor may sit at an offset inside it
    off = int(getattr(hdl, "offset", 0) or 0)
    ptrs = [p + off for p in ptrs] if off and ptrs[self.rank] + off == t.data_ptr() else ptrs
    assert ptrs[self.rank] == t.data_ptr(), "symmetric allocation does not start at the local tensor"
    mc = 0
    try:
      mc = int(hdl.multicast_ptr or 0)
      if mc and off:
        mc += off
    except Exception:  # pylint: disable=broad-except
      mc = 0
    if guard:
      lo, hi = t[:guard].view(torch.int32), t[guard + int(numel):].view(torch.int32)
      lo.fill_(self.GUARD_WORD)
      hi.fill_(self.GUARD_WORD)
      torch.cuda.synchronize(self.device)
      self._guards.append((lo, hi))
      ptrs = [p + self.GUARD_BYTES for p in ptrs]
      mc = mc + self.GUARD_BYTES if mc else 0
      t = t[guard:guard + int(numel)]
    return SymmTensor(t, ptrs, mc)

  def verify_canaries(self):
    """Raises if any guard word around a symmetric buffer of this rank changed."""
    for i, (lo, hi) in enumerate(self._guards):
      for side, g in (("below", lo), ("above", hi)):
        if not bool((g == self.GUARD_WORD).all()):
          bad = int((g != self.GUARD_WORD).nonzero()[0])
          raise RuntimeError(f"rank {self.rank}: symmetric buffer #{i} was overrun ({side} it, guard word {bad} changed)")

  # ---- epoch flags (stream ordered)
  def signal(self, slot: int) -> int:
    self.epochs[slot] += 1
    backend.ext().comm_signal(self.flags.table, slot, self.rank, self.world, self.epochs[slot])
    return self.epochs[slot]

  def wait(self, slot: int, epoch: int | None = None):
    backend.ext().comm_wait(self.flags.tensor, slot, self.world, self.epochs[slot] if epoch is None else epoch, self.wait_limit_ms)

  def barrier(self, slot: int = 0):
    """All ranks' streams reach this point before any continues (device side, no host sync)."""
    self.signal(slot)
    self.wait(slot)

  def check(self):
    st = backend.ext().kernel_status(True)
    if st != 0:
      raise CommTimeoutError(f"a device-side wait timed out (status {st}) on rank {self.rank}")
    if self.canaries:
      self.verify_canaries()
