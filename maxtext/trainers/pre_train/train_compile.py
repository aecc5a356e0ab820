from maxtext_b200.train.train_compile import main, plan  # noqa: F401

if __name__ == "__main__":
  import sys
  _rc = main()
  sys.exit(_rc if isinstance(_rc, int) else 0)
