"""`python -m maxtext.trainers.post_train.rl.train_rl <config.yml> key=value ...`: GRPO / GSPO reinforcement learning."""
from maxtext_b200.trainers.post_train.rl.train_rl import main, rl_train  # noqa: F401

if __name__ == "__main__":
  main()
