"""Resilience paths with host-made failures only: retry supervisor, uncommitted-checkpoint cleanup, preemption save,
heartbeats, rank departure between steps (gloo ranks)."""
import os
import signal
import subprocess
import sys

import pytest
import torch

from helpers import BASE_YML, tiny_config
from maxtext_b200.train import train as train_lib
from maxtext_b200.utils import elastic


class DictStore:
  def __init__(self):
    self.d = {}

  def set(self, k, v):
    self.d[k] = v.encode() if isinstance(v, str) else v

  def get(self, k):
    return self.d[k]

  def check(self, keys):
    return all(k in self.d for k in keys)


def test_supervisor_retries_then_succeeds():
  calls, cleaned = [], []

  def fn(attempt, world):
    calls.append((attempt, world))
    if attempt < 2:
      raise elastic.RankFailure("peer lost")
    return "ok"

  worlds = iter([4, 3, 3])
  sup = elastic.ElasticSupervisor(max_retries=5, timeout_seconds=1, min_world=2, cleanup=lambda: cleaned.append(1),
                                  live_world=lambda: next(worlds), sleep=lambda s: None)
  assert sup.run(fn) == "ok"
  assert calls == [(0, 4), (1, 3), (2, 3)] and len(cleaned) == 2
  assert [e["kind"] for e in sup.events.log] == ["attempt_start", "failure", "attempt_start", "failure", "attempt_start", "finished"]


def test_supervisor_gives_up_and_passes_non_retryable():
  sup = elastic.ElasticSupervisor(max_retries=1, sleep=lambda s: None)
  with pytest.raises(elastic.RankFailure):
    sup.run(lambda a, w: (_ for _ in ()).throw(elastic.RankFailure("x")))
  with pytest.raises(ValueError):
    elastic.ElasticSupervisor(max_retries=5).run(lambda a, w: (_ for _ in ()).throw(ValueError("bug")))


def test_supervisor_needs_min_world():
  sup = elastic.ElasticSupervisor(timeout_seconds=0.0, min_world=4, live_world=lambda: 2, sleep=lambda s: None)
  with pytest.raises(elastic.RankFailure):
    sup.run(lambda a, w: None)


def test_heartbeat_detects_quiet_rank():
  now = [100.0]
  st = DictStore()
  hbs = [elastic.Heartbeat(st, r, 3, clock=lambda: now[0]) for r in range(3)]
  assert hbs[0].dead_ranks(10) == []
  now[0] = 120.0
  hbs[0].beat(); hbs[2].beat()
  assert hbs[0].dead_ranks(10) == [1]
  with pytest.raises(elastic.RankFailure):
    hbs[0].raise_if_peer_dead(10)


def test_preemption_agreed_through_store():
  st = DictStore()
  a = elastic.PreemptionWatcher(st, install=False)
  b = elastic.PreemptionWatcher(st, install=False)
  assert not a.reached_preemption(3) and not b.reached_preemption(3)
  a.trigger()
  assert not a.reached_preemption(4)          # published "stop after step 5"; both ranks stop at the same step
  assert not b.reached_preemption(4)
  assert a.reached_preemption(5) and b.reached_preemption(5)


def test_failure_mid_run_resumes_from_last_committed(tmp_path, monkeypatch):
  """Attempt 0 fails at step 5 after leaving an uncommitted step directory behind; attempt 1 removes it, restores step 3
  and finishes; the final loss equals an uninterrupted run's."""
  args = ["steps=8", "checkpoint_period=2", "enable_checkpointing=true", "async_checkpointing=false", f"base_output_directory={tmp_path}",
          "run_name=el", "save_checkpoint_on_completion=false"]
  cfg = tiny_config(extra=args)
  monkeypatch.setenv("MAXTEXT_B200_INJECT_FAULT", "raise@5")
  attempts = []

  def fn(attempt, world):
    attempts.append(attempt)
    if attempt == 1:                      # a save that died half way: directory without commit marker
      os.makedirs(os.path.join(cfg.checkpoint_dir, "6", "items"))
    return train_lib.train_loop(cfg, attempt=attempt)

  sup = elastic.ElasticSupervisor(max_retries=2, sleep=lambda s: None)
  _, hist = sup.run(fn)
  assert attempts == [0, 1]
  assert hist[0]["step"] == 5 and hist[-1]["step"] == 7      # resumed after the step-4 checkpoint
  monkeypatch.delenv("MAXTEXT_B200_INJECT_FAULT")
  cfg2 = tiny_config(extra=[a.replace("run_name=el", "run_name=ref") for a in args])
  _, ref = train_lib.train_loop(cfg2)
  assert abs(hist[-1]["learning/loss"] - ref[-1]["learning/loss"]) < 1e-5


def test_sigterm_saves_and_stops(tmp_path, monkeypatch):
  cfg = tiny_config(extra=["steps=20", "checkpoint_period=1000", "enable_checkpointing=true", "async_checkpointing=false",
                           f"base_output_directory={tmp_path}", "run_name=pre", "save_checkpoint_on_completion=false"])
  monkeypatch.setenv("MAXTEXT_B200_INJECT_FAULT", "sigterm@3")
  eng, hist = train_lib.train_loop(cfg)
  assert hist[-1]["step"] == 3
  from maxtext_b200.checkpoint.manager import CheckpointManager
  assert CheckpointManager(cfg, eng).latest_step() == 3


def test_rank_departure_between_steps_is_seen_by_peers(tmp_path):
  """Two gloo ranks; rank 1 leaves between steps (exit code 17). Rank 0 learns it on the host, through the heartbeat
  keys of the store, before it launches its next step, and reports RankFailure."""
  worker = os.path.join(os.path.dirname(__file__), "elastic_worker.py")
  env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29641", WORLD_SIZE="2", MAXTEXT_B200_INJECT_FAULT="exit@2:1")
  procs = [subprocess.Popen([sys.executable, worker, str(tmp_path)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
  outs = [p.communicate(timeout=300)[0] for p in procs]
  assert procs[1].returncode == 17, outs[1][-2000:]
  assert procs[0].returncode == 0, outs[0][-2000:]
  assert "RANK_FAILURE_SEEN" in outs[0], outs[0][-2000:]


def test_rank_departure_faults_are_refused_while_peers_map_this_ranks_gpu_memory():
  """`exit` / `stall` must not take a rank away while its device buffers are mapped by peers; `raise` stays allowed."""
  import types
  import pytest
  from maxtext_b200.utils import elastic
  cuda_fused = types.SimpleNamespace(device=types.SimpleNamespace(type="cuda"), store=types.SimpleNamespace(fused=True, rs_nvls=True, symm=object()))
  cpu = types.SimpleNamespace(device=types.SimpleNamespace(type="cpu"), store=types.SimpleNamespace(fused=False, rs_nvls=False, symm=None))
  assert elastic.peer_memory_guard(cpu)() == ""
  assert "symmetric" in elastic.peer_memory_guard(cuda_fused)()
  for kind in ("exit", "stall"):
    inj = elastic.FaultInjector(f"{kind}@2", guard=elastic.peer_memory_guard(cuda_fused))
    inj.maybe_fire(1)
    with pytest.raises(elastic.FaultInjectionRefused):
      inj.maybe_fire(2)
    assert not elastic.retryable(elastic.FaultInjectionRefused("x"))
  inj = elastic.FaultInjector("raise@2", guard=elastic.peer_memory_guard(cuda_fused))
  with pytest.raises(elastic.RankFailure):
    inj.maybe_fire(2)


def test_timed_out_device_wait_becomes_a_retryable_error_before_the_step_is_saved():
  """The train loop reads the kernels' status word after each step's synchronize; a non-zero word (here from a stand-in
  extension) raises CommTimeoutError, which the supervisor retries."""
  import pytest
  from maxtext_b200.parallel.symm import CommTimeoutError
  from maxtext_b200.train.train import check_kernel_status
  from maxtext_b200.utils import elastic

  class FakeExt:
    def __init__(self, st):
      self.st, self.cleared = st, False

    def kernel_status(self, clear):
      st, self.cleared = self.st, bool(clear)
      if clear:
        self.st = 0
      return st
  ok = FakeExt(0)
  check_kernel_status("cuda:0", 0, ext=ok)
  bad = FakeExt(4)
  with pytest.raises(CommTimeoutError) as e:
    check_kernel_status("cuda:0", 3, ext=bad)
  assert "peer flag" in str(e.value) and "rank 3" in str(e.value) and bad.cleared
  assert elastic.retryable(e.value)
  check_kernel_status("cuda:0", 3, ext=bad)      # the word was cleared by the failed check
