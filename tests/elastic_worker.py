"""Child process of test_elastic_cpu.py: a 2-rank gloo training run in which one rank leaves between steps."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
sys.path.insert(0, os.path.dirname(__file__))

from helpers import tiny_config  # noqa: E402
from maxtext_b200.train import train as train_lib  # noqa: E402
from maxtext_b200.utils import elastic  # noqa: E402


def main():
  cfg = tiny_config(extra=["steps=50", "elastic_enabled=true", "elastic_timeout_seconds=3", "heartbeat_reporting_interval_in_seconds=1",
                           "ici_fsdp_parallelism=2", "jax_distributed_initialization_timeout=20", "hardware=cpu"], num_devices=2)
  try:
    train_lib.train_loop(cfg)
  except elastic.RankFailure as e:
    print("RANK_FAILURE_SEEN", e, flush=True)
    os._exit(0)      # the process group still has a dead peer: leave without a collective teardown
  except Exception as e:  # a collective that lost its peer also ends the attempt
    if elastic.retryable(e):
      print("RANK_FAILURE_SEEN (collective)", repr(e)[:200], flush=True)
      os._exit(0)
    raise


if __name__ == "__main__":
  main()
