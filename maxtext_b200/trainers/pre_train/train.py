from ...train.train import main, train_loop  # noqa: F401

if __name__ == "__main__":
  main()
