"""`python -m maxtext.trainers.post_train.distillation.save_top_k_teacher_logits`: see maxtext_b200.trainers.post_train.distillation.save_top_k_teacher_logits."""
from maxtext_b200.trainers.post_train.distillation.save_top_k_teacher_logits import main  # noqa: F401

if __name__ == "__main__":
  main()
