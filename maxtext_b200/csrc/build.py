"""In-tree build of the sm_100a kernel library (`csrc/build/maxtext_b200_C.so`).

`python -m maxtext_b200.csrc.build` compiles every .cu/.cpp of this directory for
`-gencode arch=compute_100a,code=sm_100a` with ninja through torch.utils.cpp_extension and leaves the
shared object next to the sources so that it ships with the tree. nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import glob
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "build")
EXT_NAME = "maxtext_b200_C"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xptxas", "-v", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
]


def sources() -> list[str]:
  return sorted(glob.glob(os.path.join(HERE, "*.cu")) + glob.glob(os.path.join(HERE, "*.cpp")))


def build_extension(verbose: bool = True):
  from torch.utils import cpp_extension
  os.makedirs(BUILD_DIR, exist_ok=True)
  os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 4)))
  mod = cpp_extension.load(
      name=EXT_NAME, sources=sources(), extra_cflags=["-O2", "-std=c++17"], extra_cuda_cflags=NVCC_FLAGS,
      extra_include_paths=[HERE], build_directory=BUILD_DIR, with_cuda=True, verbose=verbose)
  return mod


HOST_DIR = os.path.join(HERE, "host")
HOST_BUILD_DIR = os.path.join(HERE, "build_host")
HOST_EXT_NAME = "maxtext_b200_host"


def build_host_extension(verbose: bool = True):
  """The host-side runtime library (no CUDA): `csrc/host/*.cpp` -> `csrc/build_host/maxtext_b200_host.so`."""
  from torch.utils import cpp_extension
  os.makedirs(HOST_BUILD_DIR, exist_ok=True)
  return cpp_extension.load(name=HOST_EXT_NAME, sources=sorted(glob.glob(os.path.join(HOST_DIR, "*.cpp"))),
                            extra_cflags=["-O2", "-std=c++17"], extra_ldflags=["-lpthread"], build_directory=HOST_BUILD_DIR,
                            with_cuda=False, verbose=verbose)


HOST_ASAN_BUILD_DIR = os.path.join(HERE, "build_host_asan")
HOST_ASAN_EXT_NAME = "maxtext_b200_host_asan"


def build_host_extension_sanitized(verbose: bool = True):
  """The same host library under AddressSanitizer + UndefinedBehaviorSanitizer (`--sanitize`), as a module of its own
  (`csrc/build_host_asan/maxtext_b200_host_asan.so`). It must be loaded into a Python that has libasan pre-loaded
  (LD_PRELOAD=$(g++ -print-file-name=libasan.so), ASAN_OPTIONS=detect_leaks=0): `tests/test_native_loader_cpu.py` does that in
  a child process."""
  import subprocess
  from torch.utils import cpp_extension
  os.makedirs(HOST_ASAN_BUILD_DIR, exist_ok=True)
  # the sanitizer runtimes ship with one particular compiler installation: build with a g++ that can find its own libasan
  for cxx in (os.environ.get("CXX", ""), "g++", "/usr/bin/g++"):
    if not cxx:
      continue
    try:
      lib = subprocess.run([cxx, "-print-file-name=libasan.so"], capture_output=True, text=True, check=False).stdout.strip()
    except OSError:
      continue
    if lib and os.path.isfile(lib):
      os.environ["CXX"] = cxx
      break
  flags = ["-O1", "-g", "-std=c++17", "-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-fno-sanitize-recover=undefined"]
  return cpp_extension.load(name=HOST_ASAN_EXT_NAME, sources=sorted(glob.glob(os.path.join(HOST_DIR, "*.cpp"))), extra_cflags=flags,
                            extra_ldflags=["-lpthread", "-fsanitize=address,undefined"], build_directory=HOST_ASAN_BUILD_DIR,
                            with_cuda=False, verbose=verbose)


if __name__ == "__main__":
  if "--sanitize" in sys.argv:
    build_host_extension_sanitized(verbose="-q" not in sys.argv)
    print("built", os.path.join(HOST_ASAN_BUILD_DIR, HOST_ASAN_EXT_NAME + ".so"))
    sys.exit(0)
  build_host_extension(verbose="-q" not in sys.argv)
  build_extension(verbose="-q" not in sys.argv)
  print("built", os.path.join(BUILD_DIR, EXT_NAME + ".so"))
