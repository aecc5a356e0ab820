from maxtext_b200.inference.decode import main, decode  # noqa: F401

if __name__ == "__main__":
  main()
