"""Host-side resilience: retry supervisor, preemption watcher, heartbeats, and a fault injector for tests.

Counterpart of src/maxtext/utils/elastic_utils.py:56-281 (elastic_retry wrapper: goodput events, cleanup of a
checkpoint that has no commit marker, mesh rebuilt from the live devices, restart from the last good step) and of
the preemption save of src/maxtext/common/checkpointing.py:466,820-828. One process drives one GPU here, so "a slice
was lost" shows up as (a) an exception out of a collective or out of a bounded device wait (`CommTimeoutError`), or
(b) a rank whose heartbeat in the rendezvous store stopped. Every failure this module reacts to is visible on the
host; nothing here needs a device to fault.
"""
from __future__ import annotations

import os
import signal
import threading
import time
from dataclasses import dataclass, field

from . import max_logging


class ScaleUpSignal(Exception):
  """Raised between steps when more ranks became available: the supervisor re-initialises with the larger world."""


class FaultInjectionRefused(RuntimeError):
  """An injected rank departure was refused because it is unsafe in the current set-up (not retryable)."""


def peer_memory_guard(engine):
  """For FaultInjector: a reason string when `engine` holds peer-mapped GPU memory, else ''."""
  def guard():
    dev = getattr(engine, "device", None)
    if dev is None or getattr(dev, "type", "cpu") != "cuda":
      return ""
    store = getattr(engine, "store", None)
    if store is not None and (getattr(store, "fused", False) or getattr(store, "rs_nvls", False) or getattr(store, "symm", None) is not None):
      return "this rank's gradient / parameter buffers are symmetric memory mapped by its peers (fused communication is on)"
    if os.environ.get("NCCL_NVLS_ENABLE", "") != "0":
      return "NCCL may have bound this rank's buffers to an NVLS multicast object (set NCCL_NVLS_ENABLE=0)"
    return ""
  return guard


class RankFailure(RuntimeError):
  """A peer stopped answering (heartbeat) or a collective / device wait gave up."""


def retryable(exc: BaseException) -> bool:
  from ..parallel.symm import CommTimeoutError
  if isinstance(exc, (ScaleUpSignal, RankFailure, CommTimeoutError, ConnectionError, TimeoutError)):
    return True
  name = type(exc).__name__
  if name in ("DistBackendError", "DistNetworkError", "DistStoreError"):
    return True
  msg = str(exc)
  return isinstance(exc, RuntimeError) and any(k in msg for k in ("NCCL", "ProcessGroup", "Connection closed", "Connection reset", "Broken pipe", "timed out", "Timed out"))


@dataclass
class ElasticEvents:
  """What happened, in order; mirrors the goodput events the reference records around a retry."""
  log: list = field(default_factory=list)

  def add(self, kind: str, **kw):
    self.log.append({"t": time.time(), "kind": kind, **kw})
    max_logging.log(f"[elastic] {kind} {kw}")


class ElasticSupervisor:
  """Runs `fn(attempt, world_hint)` until it returns, retrying on failures that a smaller / larger world can survive.

  `cleanup` runs before every retry (tear down process groups, drop an uncommitted checkpoint);
  `live_world` reports how many ranks can take part in the next attempt; fewer than `min_world` ends the job.
  Keys: elastic_enabled, elastic_max_retries, elastic_timeout_seconds, elastic_min_slice_count.
  """

  def __init__(self, max_retries: int = 10, timeout_seconds: float = 300.0, min_world: int = 1, cleanup=None, live_world=None,
               sleep=time.sleep):
    self.max_retries, self.timeout, self.min_world = int(max_retries), float(timeout_seconds), int(min_world)
    self.cleanup, self.live_world, self.sleep = cleanup, live_world, sleep
    self.events = ElasticEvents()

  @classmethod
  def from_config(cls, config, **kw):
    mw = config.elastic_min_slice_count if config.elastic_min_slice_count > 0 else 1
    return cls(config.elastic_max_retries, config.elastic_timeout_seconds, mw, **kw)

  def _wait_for_world(self) -> int | None:
    if self.live_world is None:
      return None
    t0 = time.time()
    while True:
      n = int(self.live_world())
      if n >= self.min_world:
        return n
      if time.time() - t0 > self.timeout:
        raise RankFailure(f"only {n} ranks alive after {self.timeout}s, need {self.min_world}")
      self.sleep(min(1.0, self.timeout / 10))

  def run(self, fn):
    attempt = 0
    world = self._wait_for_world()
    while True:
      try:
        self.events.add("attempt_start", attempt=attempt, world=world)
        out = fn(attempt, world)
        self.events.add("finished", attempt=attempt)
        return out
      except BaseException as e:  # pylint: disable=broad-except
        if not retryable(e) or attempt >= self.max_retries:
          self.events.add("giving_up", attempt=attempt, error=repr(e))
          raise
        self.events.add("scale_up" if isinstance(e, ScaleUpSignal) else "failure", attempt=attempt, error=repr(e))
        if self.cleanup is not None:
          self.cleanup()
        attempt += 1
        world = self._wait_for_world()


def teardown_distributed():
  """Abort-style cleanup between attempts: the process group of a failed attempt may have collectives outstanding."""
  import torch.distributed as dist
  if dist.is_available() and dist.is_initialized():
    try:
      dist.destroy_process_group()
    except Exception as e:  # pylint: disable=broad-except
      max_logging.log(f"[elastic] destroy_process_group: {e!r}")


# ----------------------------------------------------------------------------------------------- preemption
class PreemptionWatcher:
  """SIGTERM (the scheduler's notice) -> `reached_preemption()` turns True on every rank at the same step.

  Ranks agree through the rendezvous store: the rank that got the signal publishes `preempt_at = step + 1`, every
  rank reads the key once per step (a host-side lookup; no collective is launched).
  """
  KEY = "maxtext_b200/preempt_at"

  def __init__(self, store=None, signals=(signal.SIGTERM,), install: bool = True):
    self._flag = threading.Event()
    self.store = store
    self._published = False
    self._old = {}
    if install and threading.current_thread() is threading.main_thread():
      for s in signals:
        self._old[s] = signal.signal(s, self._on_signal)

  def _on_signal(self, signum, frame):  # pylint: disable=unused-argument
    self._flag.set()

  def trigger(self):
    self._flag.set()

  def reached_preemption(self, step: int) -> bool:
    if self.store is None:
      return self._flag.is_set()
    if self._flag.is_set() and not self._published:
      self.store.set(self.KEY, str(step + 1))
      self._published = True
    try:
      if not self.store.check([self.KEY]):
        return False
      return step >= int(self.store.get(self.KEY))
    except Exception:  # pylint: disable=broad-except
      return self._flag.is_set()

  def close(self):
    for s, h in self._old.items():
      signal.signal(s, h)


# ----------------------------------------------------------------------------------------------- heartbeats
class Heartbeat:
  """Each rank writes `hb/<rank>` = wall time from a daemon thread; `dead_ranks` lists ranks that went quiet.

  The role of src/maxtext/common/gcp_workload_monitor.py (heartbeat thread) with the rendezvous store in place of
  Cloud Monitoring.
  """

  def __init__(self, store, rank: int, world: int, interval: float = 5.0, clock=time.time):
    self.store, self.rank, self.world, self.interval, self.clock = store, rank, world, interval, clock
    self._stop = threading.Event()
    self._thread = None
    self.t0 = clock()
    self.beat()

  def beat(self):
    self.store.set(f"hb/{self.rank}", repr(self.clock()))

  def start(self):
    def loop():
      while not self._stop.wait(self.interval):
        try:
          self.beat()
        except Exception:  # pylint: disable=broad-except
          return
    self._thread = threading.Thread(target=loop, daemon=True, name="heartbeat")
    self._thread.start()
    return self

  def leave(self):
    """Announce an orderly departure (between steps): peers see it at their next check, without waiting for a timeout."""
    self.stop()
    self.store.set(f"bye/{self.rank}", "1")

  def dead_ranks(self, timeout: float) -> list[int]:
    now, dead = self.clock(), []
    for r in range(self.world):
      k = f"hb/{r}"
      if self.store.check([f"bye/{r}"]):
        dead.append(r)
        continue
      if not self.store.check([k]):
        if now - self.t0 > timeout:       # never showed up
          dead.append(r)
        continue
      if now - float(self.store.get(k).decode()) > timeout:
        dead.append(r)
    return dead

  def raise_if_peer_dead(self, timeout: float):
    d = [r for r in self.dead_ranks(timeout) if r != self.rank]
    if d:
      raise RankFailure(f"ranks {d} sent no heartbeat for {timeout}s")

  def stop(self):
    self._stop.set()


# ----------------------------------------------------------------------------------------------- fault injection
class FaultInjector:
  """Host-made failures for tests and drills (the role of benchmarks/disruption_management/disruption_handler.py:42-135).

  Spec `"<kind>@<step>[:rank]"`, kinds: `raise` (RankFailure out of the step loop), `sigterm` (preemption notice to
  this process), `exit` (the rank leaves between steps, exit code 17), `stall` (stops heartbeats and sleeps).
  Reads MAXTEXT_B200_INJECT_FAULT when no spec is given. Nothing here touches a device.

  `exit` and `stall` take a rank away while its peers keep running. They refuse to fire (FaultInjectionRefused) when
  `guard()` says the process holds peer-mapped device memory (symmetric buffers of the fused communication path, which may
  be bound to an NVSwitch multicast object): a rank that disappears with such mappings alive raises NVLink faults on the
  other GPUs. Use them with gloo ranks on CPU, or with `use_fused_comm_kernels=false` and NVLS off.
  """

  def __init__(self, spec: str | None = None, rank: int = 0, guard=None):
    self.guard = guard
    spec = spec if spec is not None else os.environ.get("MAXTEXT_B200_INJECT_FAULT", "")
    self.kind, self.step, self.fired = None, -1, False
    if spec:
      kind, rest = spec.split("@")
      step, _, r = rest.partition(":")
      if not r or int(r) == rank:
        self.kind, self.step = kind, int(step)

  def maybe_fire(self, step: int, attempt: int = 0, heartbeat: Heartbeat | None = None):
    if self.kind is None or self.fired or attempt > 0 or step != self.step:
      return
    if self.kind in ("exit", "stall") and self.guard is not None:
      why = self.guard()
      if why:
        raise FaultInjectionRefused(f"fault '{self.kind}' not injected: {why}")
    self.fired = True
    if self.kind == "raise":
      raise RankFailure(f"injected failure at step {step}")
    if self.kind == "sigterm":
      os.kill(os.getpid(), signal.SIGTERM)
    elif self.kind == "exit":
      if heartbeat is not None:
        heartbeat.leave()
      os._exit(17)
    elif self.kind == "stall":
      if heartbeat is not None:
        heartbeat.stop()
      time.sleep(3600)
