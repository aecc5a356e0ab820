"""The allocation-free sum-of-squares entry point, called the way an embedder would: through its exported C
symbol with raw device pointers. Some hosts of this library may not allocate device memory while they run
(graph replay loops, allocators that hold a lock, fixed memory budgets), so `mt_sumsq_noalloc` keeps its scratch
inside the library image. The test checks it against the regular entry point (caller-provided scratch) on two
calls in a row, the second on different data and a different length, which also shows that nothing left in the
shared scratch by the first call leaks into the second. This file sorts last on purpose."""
import ctypes
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
  from maxtext_b200.ops import backend
  backend.ext(required=True)           # makes sure the library is built and its dependencies are loaded
  lib = ctypes.CDLL(backend.so_path())
  lib.mt_sumsq_noalloc.restype = ctypes.c_int
  lib.mt_sumsq_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
  lib.mt_sumsq_noalloc_strerror.restype = ctypes.c_char_p
  lib.mt_sumsq_noalloc_strerror.argtypes = [ctypes.c_int]
  lib.mt_sumsq.restype = ctypes.c_int
  lib.mt_sumsq.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
  lib.mt_sumsq_num_partials.restype = ctypes.c_int
  lib.mt_sumsq_num_partials.argtypes = [ctypes.c_long, ctypes.c_int]
  return lib


def test_no_alloc_sumsq_matches_regular_entry_point_twice():
  lib = _lib()
  dev = torch.device("cuda", torch.cuda.current_device())
  sms = torch.cuda.get_device_properties(dev).multi_processor_count
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  g = torch.Generator(device="cuda").manual_seed(1234)
  calls = 0
  for n, scale in ((3_000_003, 1.0), (517_001, 7.5)):
    x = scale * torch.randn(n, device=dev, generator=g)
    # regular entry point: the caller brings the scratch
    parts = lib.mt_sumsq_num_partials(n, sms)
    scratch = torch.empty(parts, device=dev)
    want = torch.zeros(1, device=dev)
    assert lib.mt_sumsq(x.data_ptr(), n, scratch.data_ptr(), want.data_ptr(), sms, stream) == 0
    # allocation-free entry point: inputs and outputs only
    got = torch.zeros(1, device=dev)
    gc.collect()                       # garbage of earlier tests must not be freed between the two readings
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    free_before = torch.cuda.mem_get_info(dev)[0]
    rc = lib.mt_sumsq_noalloc(x.data_ptr(), n, got.data_ptr(), stream)
    assert rc == 0, lib.mt_sumsq_noalloc_strerror(rc).decode()
    assert torch.cuda.memory_allocated(dev) <= before, "the allocation-free entry point allocated through torch"
    torch.cuda.synchronize()
    if calls > 0:
      # torch's counter only sees torch's allocator; the driver's free-memory figure also sees a cudaMalloc made by the
      # library itself. Checked from the second call on: the first may load the module's kernels into the context.
      assert torch.cuda.mem_get_info(dev)[0] >= free_before, "device memory shrank during an allocation-free call"
    calls += 1
    ref = x.double().pow(2).sum().item()
    assert abs(got.item() - want.item()) <= 1e-6 * abs(want.item())
    assert abs(got.item() - ref) <= 1e-4 * ref


def test_no_alloc_sumsq_rejects_oversized_and_bad_input():
  lib = _lib()
  x = torch.ones(16, device="cuda")
  out = torch.zeros(1, device="cuda")
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  too_long = (1 << 36) + 1
  rc = lib.mt_sumsq_noalloc(x.data_ptr(), too_long, out.data_ptr(), stream)
  assert rc == -2 and b"MT_SUMSQ_NOALLOC_MAX_ELEMS" in lib.mt_sumsq_noalloc_strerror(rc)
  assert lib.mt_sumsq_noalloc(None, 16, out.data_ptr(), stream) == -1
  torch.cuda.synchronize()
  assert out.item() == 0.0
