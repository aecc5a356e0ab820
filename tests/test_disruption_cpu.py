"""Disruption harness on two gloo ranks: a pre-emption notice and a killed rank; the job restarts and finishes every step."""
import os
import sys

import pytest

from helpers import BASE_YML, ROOT, TINY


def _cmd(tmp_path, steps):
  base = [a for a in TINY if not a.startswith(("enable_checkpointing", "steps", "per_device_batch_size"))]
  return [sys.executable, "-m", "maxtext_b200.train.train", BASE_YML] + base + [
      "model_name=llama3-8b", f"base_output_directory={tmp_path}", "run_name=job", f"steps={steps}", "enable_checkpointing=true",
      "checkpoint_period=2", "async_checkpointing=false", "per_device_batch_size=2", "ici_fsdp_parallelism=2",
      f"learning_rate_schedule_steps={steps}"]


def test_trigger_rules_and_log_monitor(tmp_path):
  import time
  from maxtext_b200.benchmarks.disruption_management import Disruption, StepMonitor
  d = Disruption("a", "step", 3)
  assert not d.due(2, 100.0) and d.due(3, 0.0)
  t = Disruption("b", "time", 1.5)
  assert not t.due(50, 1.0) and t.due(-1, 2.0)
  d.fired["step"] = 3
  assert not d.due(9, 0.0)                      # fires once
  with pytest.raises(ValueError):
    Disruption("c", "moon", 1)
  with pytest.raises(ValueError):
    Disruption("c", "step", 1, method="unplug")
  log = tmp_path / "r0.log"
  mon = StepMonitor(str(log), poll=0.01)
  mon.start()
  with open(log, "w") as fh:
    fh.write("hello\ncompleted step: 0, seconds: 1\ncompleted st")
    fh.flush()
    time.sleep(0.1)
    assert mon.last_step == 0
    fh.write("ep: 1, seconds\ncompleted step: 2 x\n")
    fh.flush()
    time.sleep(0.1)
  mon.stop()
  mon.join(1)
  assert [s for s, _ in mon.steps] == [0, 1, 2]


def test_job_survives_a_preemption_notice_and_a_killed_rank(tmp_path):
  from maxtext_b200.benchmarks.disruption_management import Disruption, DisruptionManager
  steps = 12
  ds = [Disruption("notice", "step", 3, "sigterm", "all"), Disruption("crash", "step", 8, "sigkill", 1)]
  env = {"MAXTEXT_B200_QUIET": "0", "OMP_NUM_THREADS": "2", "CUDA_VISIBLE_DEVICES": ""}
  rep = DisruptionManager(_cmd(tmp_path, steps), 2, steps, str(tmp_path / "logs"), ds, max_restarts=4, grace=5.0, env=env, cwd=ROOT).run()
  assert rep["completed"] and rep["final_step"] == steps - 1, rep
  assert rep["restarts"] >= 2 and [d["name"] for d in rep["disruptions"]] == ["notice", "crash"], rep
  notice, crash = rep["disruptions"]
  # the notice makes every rank save and leave cleanly: the next attempt continues after the agreed stop step, nothing is lost
  assert rep["attempts"][notice["attempt"]]["return_codes"] == [0, 0]
  assert notice["resumed_from_step"] > notice["step"] - 1 and notice["lost_steps"] <= 1, rep
  assert notice["resumed_from_step"] == rep["attempts"][notice["attempt"]]["last_step"] + 1, rep          # nothing repeated, nothing skipped
  # the crash loses at most the steps since the last checkpoint (period 2)
  # (the signal lands a little after the step the monitor saw: the attempt may have finished another step or two by then)
  assert crash["resumed_from_step"] <= rep["attempts"][crash["attempt"]]["last_step"] + 1 and crash["lost_steps"] <= 3, rep
  assert crash["recovery_seconds"] > 0, rep
  assert os.path.isfile(tmp_path / "logs" / "disruption_report.json")
