"""Alias of `maxtext_b200.inference.maxengine_server` under the module path the reference uses."""
from maxtext_b200.inference.maxengine_server import *  # noqa: F401,F403
from maxtext_b200.inference.maxengine_server import main  # noqa: F401

if __name__ == "__main__":
  import sys
  _rc = main()
  sys.exit(_rc if isinstance(_rc, int) else 0)
