"""The C++ batch producer: packing rules, rank sharding, .npy and raw files, exact resume, agreement with a Python model."""
import numpy as np
import pytest
import torch

from maxtext_b200.input_pipeline.native_loader import NativeTokenIterator, host_lib

EOS = 1


def _docs(rng, n, lo=2, hi=12):
  return [list(rng.integers(2, 100, size=int(rng.integers(lo, hi)))) + [EOS] for _ in range(n)]


def _python_batches(docs, seq, batch, rank, world, n_batches):
  """The packing rule restated in Python: documents of the rank in order, next-fit rows, long ones cut with one token overlap."""
  pieces = []
  for d_i, d in enumerate(docs):
    if d_i % world != rank or len(d) < 2:
      continue
    while len(d) > seq + 1:
      pieces.append(d[:seq + 1])
      d = d[seq:]
    if len(d) >= 2:
      pieces.append(d)
  out, k = [], 0
  for _ in range(n_batches):
    inp, tgt, seg = np.zeros((batch, seq), np.int32), np.zeros((batch, seq), np.int32), np.zeros((batch, seq), np.int32)
    for r in range(batch):
      used, s = 0, 0
      while used < seq and k < len(pieces):
        p = pieces[k]
        if len(p) - 1 > seq - used and used > 0:
          break
        s += 1
        take = min(len(p) - 1, seq - used)
        inp[r, used:used + take], tgt[r, used:used + take], seg[r, used:used + take] = p[:take], p[1:take + 1], s
        used += take
        k += 1
    out.append((inp, tgt, seg))
  return out


@pytest.fixture(scope="module")
def lib():
  try:
    return host_lib()
  except Exception as e:  # pylint: disable=broad-except
    pytest.skip(f"host library cannot be built here: {e}")


def test_packing_matches_python_model_and_shards_by_rank(lib, tmp_path):
  rng = np.random.default_rng(0)
  docs = _docs(rng, 200) + [list(rng.integers(2, 100, size=40)) + [EOS]]           # one document longer than a row
  flat = np.array([t for d in docs for t in d], dtype=np.int32)
  a, b = str(tmp_path / "a.npy"), str(tmp_path / "b.bin")
  cut = sum(len(d) for d in docs[:120])
  np.save(a, flat[:cut])
  flat[cut:].tofile(b)
  for rank, world in ((0, 1), (0, 2), (1, 2)):
    it = NativeTokenIterator([a, b], 16, 3, EOS, rank, world, pin=False)
    want = _python_batches(docs, 16, 3, rank, world, 6)
    for inp, tgt, seg in want:
      got = next(it)
      assert np.array_equal(got["inputs"].numpy(), inp) and np.array_equal(got["targets"].numpy(), tgt)
      assert np.array_equal(got["inputs_segmentation"].numpy(), seg)
      pos = got["inputs_position"].numpy()
      assert (pos[seg == 0] == 0).all() and all(pos[r, c] == (0 if c == 0 or seg[r, c] != seg[r, c - 1] else pos[r, c - 1] + 1)
                                                 for r in range(3) for c in range(16) if seg[r, c])


def test_state_and_seek_resume_exactly_and_epochs_wrap(lib, tmp_path):
  rng = np.random.default_rng(1)
  docs = _docs(rng, 30)
  p = str(tmp_path / "t.bin")
  np.array([t for d in docs for t in d], dtype=np.int32).tofile(p)
  it = NativeTokenIterator([p], 8, 2, EOS, pin=False)
  for _ in range(5):
    next(it)
  st = it.state()
  after = [{k: v.clone() for k, v in next(it).items()} for _ in range(40)]          # runs through several epochs
  assert it.state()["native_position"][3] >= 1
  it2 = NativeTokenIterator([p], 8, 2, EOS, pin=False)
  it2.load_state(st)
  for want in after:
    got = next(it2)
    assert all(torch.equal(got[k], want[k]) for k in want)


def test_bad_inputs_are_reported(lib, tmp_path):
  p = str(tmp_path / "e.bin")
  np.array([EOS, EOS, EOS], dtype=np.int32).tofile(p)
  with pytest.raises(RuntimeError):
    NativeTokenIterator([p], 8, 2, EOS, pin=False)
  with pytest.raises(RuntimeError):
    NativeTokenIterator([str(tmp_path / "missing.bin")], 8, 2, EOS, pin=False)


def test_train_cli_reads_token_files_through_the_native_loader(lib, tmp_path):
  import os
  from helpers import TINY, BASE_YML
  from maxtext_b200.train import train as T
  rng = np.random.default_rng(2)
  docs = _docs(rng, 400, 4, 40)
  np.array([t for d in docs for t in d], dtype=np.int32).tofile(str(tmp_path / "train.bin"))
  args = [a for a in TINY if not a.startswith(("dataset_type", "steps", "learning_rate="))] + [
      "dataset_type=tokens", f"dataset_path={tmp_path}/*.bin", "tokenizer_type=byte", "steps=4", f"base_output_directory={tmp_path}",
      "run_name=tok", "learning_rate=3e-3"]
  eng, hist = T.main(["train", BASE_YML] + args)
  assert len(hist) == 4 and hist[-1]["learning/loss"] < hist[0]["learning/loss"] + 0.5 and all(np.isfinite(h["learning/loss"]) for h in hist)


def test_loader_under_address_and_undefined_behaviour_sanitizers(tmp_path):
  """The host library rebuilt with -fsanitize=address,undefined and driven in a child Python that pre-loads libasan: batches,
  epoch wrap-around, seek and shutdown with a full queue must not trip either sanitizer."""
  import os
  import subprocess
  import sys
  asan = subprocess.run(["g++", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
  if not asan or not os.path.isfile(asan):
    pytest.skip("libasan is not installed")
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  rng = np.random.default_rng(0)
  toks = np.concatenate([np.asarray(d, dtype=np.int32) for d in _docs(rng, 40)])
  f = tmp_path / "a.bin"
  toks.tofile(f)
  code = f"""
import sys, torch
sys.path.insert(0, {root!r})
from maxtext_b200.csrc import build
m = build.build_host_extension_sanitized(verbose=False)
L = m.TokenLoader([{str(f)!r}], 16, 2, {EOS}, 0, 1, 3)
bufs = [torch.zeros(2, 16, dtype=torch.int32) for _ in range(4)]
seen = []
for i in range(40):                      # several passes over the file
  L.next(*bufs)
  seen.append(bufs[0].clone())
st = L.state()
L.next(*bufs); a = bufs[0].clone()
L.seek(list(st))
L.next(*bufs)
assert torch.equal(a, bufs[0]), "seek did not reproduce the batch"
del L                                    # the worker is blocked on a full queue: the destructor must wake and join it
print("sanitized-ok")
"""
  env = dict(os.environ, LD_PRELOAD=asan, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1", CUDA_VISIBLE_DEVICES="")
  r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=900)
  assert r.returncode == 0 and "sanitized-ok" in r.stdout, (r.stdout[-1500:], r.stderr[-3000:])
  assert "runtime error" not in r.stderr and "AddressSanitizer" not in r.stderr, r.stderr[-3000:]
