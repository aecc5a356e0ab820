"""`python -m maxtext.trainers.post_train.distillation.train_distill`: see maxtext_b200.trainers.post_train.distillation.train_distill."""
from maxtext_b200.trainers.post_train.distillation.train_distill import main  # noqa: F401

if __name__ == "__main__":
  main()
