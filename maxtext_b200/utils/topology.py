"""Named target topologies for plan-only (no device) compilation runs.

The reference maps TPU slice names to chip counts (src/maxtext/utils/accelerator_to_spec_map.py);
here the names describe NVLink domains: `b200-8` is one HGX box, `b200-8x4` four of them.
"""
import re


def devices_in(name: str) -> int:
  m = re.fullmatch(r"(?:[a-z0-9]+)-(\d+)(?:x(\d+))?", name.strip().lower())
  if not m:
    raise ValueError(f"unknown compile_topology {name!r}; expected e.g. b200-8 or v5e-256")
  n = int(m.group(1))
  return n * int(m.group(2)) if m.group(2) else n
