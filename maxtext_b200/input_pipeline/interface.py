"""Dataset dispatch by `dataset_type` (src/maxtext/input_pipeline/input_pipeline_interface.py:34-120)."""
from __future__ import annotations


def create_data_iterator(config, data_rank: int = 0, data_world: int = 1, split: str = "train"):
  t = config.dataset_type
  if t == "synthetic":
    from .synthetic import SyntheticDataIterator
    return SyntheticDataIterator(config, data_rank, data_world)
  if t in ("hf", "grain", "tfds", "c4_mlperf", "olmo_grain"):
    from .file_pipeline import create_file_iterator
    return create_file_iterator(config, data_rank, data_world, split)
  raise ValueError(f"unknown dataset_type {t}")
