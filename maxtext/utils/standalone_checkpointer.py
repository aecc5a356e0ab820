"""Alias of `maxtext_b200.utils.standalone_checkpointer` under the module path the reference uses."""
from maxtext_b200.utils.standalone_checkpointer import *  # noqa: F401,F403
from maxtext_b200.utils.standalone_checkpointer import main  # noqa: F401

if __name__ == "__main__":
  import sys
  _rc = main()
  sys.exit(_rc if isinstance(_rc, int) else 0)
