from maxtext_b200.train.train_compile import main, plan  # noqa: F401

if __name__ == "__main__":
  import sys
  sys.exit(main())
