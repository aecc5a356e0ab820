"""Job-level disruption manager.

  Disruption(name, trigger_type="step" | "time", trigger_value, method="sigterm" | "sigkill", target_rank=int | "all")

The manager starts `world` rank processes of a training command (one per GPU; gloo ranks on a CPU box), follows rank 0's log
for `completed step: N` lines (`StepMonitor`), and when a disruption's trigger is met signals its target:

  sigterm  the pre-emption notice: the trainer's watcher agrees on a stop step across ranks, saves, and every rank exits 0
  sigkill  a crashed rank: its peers fail on their next collective (or are stopped by the manager after `grace` seconds)

After the job has stopped it is launched again with the same command (same run name, so it resumes from the last committed
checkpoint), until the configured number of steps is done or `max_restarts` is used up. Faults are made on the host only:
a rank is signalled between the manager's polls, never from inside a kernel.

The report lists, per disruption: the step and time it fired, the step the next attempt resumed from, the steps lost
(finished before the disruption but after the last checkpoint), and the seconds from the signal to the first step
completed after the restart.
"""
from __future__ import annotations

import json
import os
import re
import signal
import socket
import subprocess
import sys
import threading
import time
from dataclasses import dataclass, field

STEP_RE = re.compile(r"completed step: (\d+)")


@dataclass
class Disruption:
  name: str
  trigger_type: str = "step"          # "step": after that step has completed; "time": seconds after the attempt started
  trigger_value: float = 0
  method: str = "sigterm"
  target_rank: int | str = 0          # a rank, or "all"
  fired: dict = field(default_factory=dict)

  def __post_init__(self):
    if self.trigger_type not in ("step", "time"):
      raise ValueError(f"trigger_type must be 'step' or 'time', got {self.trigger_type!r}")
    if self.method not in ("sigterm", "sigkill"):
      raise ValueError(f"method must be 'sigterm' or 'sigkill', got {self.method!r}")

  def due(self, step: int, elapsed: float) -> bool:
    return not self.fired and (step >= self.trigger_value if self.trigger_type == "step" else elapsed >= self.trigger_value)


class StepMonitor(threading.Thread):
  """Follows a growing log file; `steps` holds (step, wall time) of every `completed step` line seen so far."""

  def __init__(self, path: str, poll: float = 0.05):
    super().__init__(daemon=True)
    self.path, self.poll = path, poll
    self.steps: list[tuple[int, float]] = []
    self._stop_flag = threading.Event()

  @property
  def last_step(self) -> int:
    return self.steps[-1][0] if self.steps else -1

  def run(self):
    pos = 0
    while not self._stop_flag.is_set():
      try:
        with open(self.path, "r", errors="replace") as fh:
          fh.seek(pos)
          chunk = fh.read()
          # only whole lines are consumed; a partial last line is read again next time
          cut = chunk.rfind("\n") + 1
          pos += len(chunk[:cut].encode(errors="replace"))
          for m in STEP_RE.finditer(chunk[:cut]):
            self.steps.append((int(m.group(1)), time.time()))
      except FileNotFoundError:
        pass
      time.sleep(self.poll)

  def stop(self):
    self._stop_flag.set()


def _free_port() -> int:
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


class DisruptionManager:
  def __init__(self, argv: list[str], world: int, total_steps: int, log_dir: str, disruptions: list[Disruption], max_restarts: int = 4,
               grace: float = 20.0, env: dict | None = None, cwd: str | None = None, attempt_timeout: float = 600.0):
    self.argv, self.world, self.total_steps, self.log_dir = list(argv), int(world), int(total_steps), log_dir
    self.disruptions, self.max_restarts, self.grace = list(disruptions), int(max_restarts), float(grace)
    self.env, self.cwd, self.attempt_timeout = dict(env or {}), cwd, float(attempt_timeout)
    os.makedirs(log_dir, exist_ok=True)

  def _start(self, attempt: int):
    port = _free_port()
    procs, logs = [], []
    for r in range(self.world):
      env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(self.world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
      env.update(self.env)
      path = os.path.join(self.log_dir, f"attempt{attempt}_rank{r}.log")
      fh = open(path, "wb")
      procs.append(subprocess.Popen(self.argv, cwd=self.cwd, env=env, stdout=fh, stderr=subprocess.STDOUT))
      logs.append((path, fh))
    return procs, logs

  def _signal(self, procs, d: Disruption):
    sig = signal.SIGTERM if d.method == "sigterm" else signal.SIGKILL
    targets = range(self.world) if d.target_rank == "all" else [int(d.target_rank)]
    for r in targets:
      if procs[r].poll() is None:
        procs[r].send_signal(sig)            # the exact process this manager started

  def run(self) -> dict:
    events, attempts = [], []
    done_step = -1
    pending = None                            # the disruption whose recovery is being timed
    for attempt in range(self.max_restarts + 1):
      procs, logs = self._start(attempt)
      mon = StepMonitor(logs[0][0])
      mon.start()
      t0 = time.time()
      killed_at = None
      while any(p.poll() is None for p in procs):
        now = time.time()
        if pending is not None and mon.steps and pending.fired["attempt"] != attempt:
          first = mon.steps[0]
          pending.fired.update(resumed_from_step=first[0], recovery_seconds=round(first[1] - pending.fired["time"], 3),
                               lost_steps=max(0, pending.fired["step"] - first[0] + 1))
          pending = None
        for d in self.disruptions:
          if d.due(mon.last_step, now - t0) and any(p.poll() is None for p in procs):
            self._signal(procs, d)
            d.fired.update(step=mon.last_step, time=now, attempt=attempt)
            events.append(d)
            pending = d
            if d.method == "sigkill":
              killed_at = now
        if killed_at is not None and now - killed_at > self.grace:
          for p in procs:                     # peers that did not notice the missing rank by themselves
            if p.poll() is None:
              p.kill()
        if now - t0 > self.attempt_timeout:
          for p in procs:
            if p.poll() is None:
              p.kill()
        time.sleep(0.05)
      time.sleep(0.2)                         # let the monitor read the tail of the log
      mon.stop()
      mon.join(timeout=2)
      for _, fh in logs:
        fh.close()
      codes = [p.returncode for p in procs]
      if pending is not None and mon.steps and "resumed_from_step" not in pending.fired and pending.fired.get("attempt") != attempt:
        first = mon.steps[0]
        pending.fired.update(resumed_from_step=first[0], recovery_seconds=round(first[1] - pending.fired["time"], 3),
                             lost_steps=max(0, pending.fired["step"] - first[0] + 1))
        pending = None
      done_step = max(done_step, mon.last_step)
      attempts.append({"attempt": attempt, "return_codes": codes, "first_step": mon.steps[0][0] if mon.steps else None,
                       "last_step": mon.last_step, "seconds": round(time.time() - t0, 3)})
      if done_step >= self.total_steps - 1 and all(c == 0 for c in codes):
        break
    report = {"completed": done_step >= self.total_steps - 1, "final_step": done_step, "restarts": len(attempts) - 1, "attempts": attempts,
              "disruptions": [{"name": d.name, "method": d.method, "trigger": f"{d.trigger_type}={d.trigger_value}", "target_rank": d.target_rank,
                               **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in d.fired.items()}} for d in events]}
    with open(os.path.join(self.log_dir, "disruption_report.json"), "w") as fh:
      json.dump(report, fh, indent=1)
    return report


def main(argv=None):
  """python -m maxtext_b200.benchmarks.disruption_management.disruption_manager --world 2 --steps 20 --log-dir /tmp/d \\
       --disrupt pre:step:5:sigterm:all --disrupt crash:step:12:sigkill:1 -- <training command with checkpointing on>"""
  import argparse
  ap = argparse.ArgumentParser()
  ap.add_argument("--world", type=int, default=1)
  ap.add_argument("--steps", type=int, required=True)
  ap.add_argument("--log-dir", required=True)
  ap.add_argument("--max-restarts", type=int, default=4)
  ap.add_argument("--disrupt", action="append", default=[], help="name:step|time:value:sigterm|sigkill:rank|all")
  ap.add_argument("command", nargs=argparse.REMAINDER)
  a = ap.parse_args(argv)
  ds = []
  for spec in a.disrupt:
    name, tt, val, method, target = spec.split(":")
    ds.append(Disruption(name, tt, float(val), method, target if target == "all" else int(target)))
  cmd = a.command[1:] if a.command and a.command[0] == "--" else a.command
  rep = DisruptionManager(cmd, a.world, a.steps, a.log_dir, ds, a.max_restarts).run()
  print(json.dumps(rep, indent=1))
  return 0 if rep["completed"] else 1


if __name__ == "__main__":
  sys.exit(main())
