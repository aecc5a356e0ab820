"""`python -m maxtext.trainers.tokenizer.train_tokenizer`: SentencePiece vocabulary trainer."""
from maxtext_b200.trainers.tokenizer.train_tokenizer import main, train_tokenizer  # noqa: F401

if __name__ == "__main__":
  main()
