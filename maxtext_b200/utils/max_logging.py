"""Rank-aware logging helpers (the role of src/maxtext/utils/max_logging.py)."""
import logging
import os
import sys

_logger = logging.getLogger("maxtext_b200")
if not _logger.handlers:
  class _Stdout(logging.StreamHandler):
    """Always writes to the current sys.stdout (which test harnesses and launchers may swap)."""
    def emit(self, record):
      self.stream = sys.stdout
      super().emit(record)

  _h = _Stdout(sys.stdout)
  _h.setFormatter(logging.Formatter("%(message)s"))
  _logger.addHandler(_h)
  _logger.setLevel(os.environ.get("MAXTEXT_B200_LOGLEVEL", "INFO"))
  _logger.propagate = False


def _rank():
  return int(os.environ.get("RANK", "0"))


def log(msg, all_ranks=False):
  if all_ranks or _rank() == 0:
    _logger.info(msg)


info = log


def debug(msg):
  if _rank() == 0:
    _logger.debug(msg)


def warning(msg):
  _logger.warning(f"[rank {_rank()}] WARNING: {msg}")


def error(msg):
  _logger.error(f"[rank {_rank()}] ERROR: {msg}")
