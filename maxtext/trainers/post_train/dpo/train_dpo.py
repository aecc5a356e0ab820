"""`python -m maxtext.trainers.post_train.dpo.train_dpo <config.yml> key=value ...`: the training loop with `use_dpo=true`
(chosen / rejected pairs against a frozen copy of the starting policy; src/maxtext/trainers/post_train/dpo/train_dpo.py)."""
import sys

from maxtext_b200.train.train import main as _train_main


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  return _train_main(argv + ["use_dpo=true"] + ([] if any(a.startswith("packing=") for a in argv) else ["packing=false"]))


if __name__ == "__main__":
  main()
