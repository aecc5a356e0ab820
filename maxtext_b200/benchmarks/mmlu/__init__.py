"""MMLU multiple-choice evaluation through the decode engine (benchmarks/mmlu/mmlu_eval.py in the reference)."""
