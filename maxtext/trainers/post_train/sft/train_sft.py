"""`python -m maxtext.trainers.post_train.sft.train_sft <config.yml> key=value ...`: the training loop with `use_sft=true`
(prompt / completion columns or chat messages; src/maxtext/trainers/post_train/sft/train_sft.py)."""
import sys

from maxtext_b200.train.train import main as _train_main


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  return _train_main(argv + ["use_sft=true"])


if __name__ == "__main__":
  main()
