"""Alias of `maxtext_b200.inference.decode_multi` under the reference's module path."""
from maxtext_b200.inference.decode_multi import *  # noqa: F401,F403
from maxtext_b200.inference.decode_multi import main

if __name__ == "__main__":
  main()
