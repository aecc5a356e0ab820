from maxtext_b200.train.train import cli, main, train_loop  # noqa: F401

if __name__ == "__main__":
  cli()
