"""Evaluation: datasets, scorers, and runners for generation, multiple-choice and perplexity tasks
(the role of src/maxtext/eval/: runner/, datasets/, scoring/, reporting/)."""
from .datasets import DATASETS, EvalSample, load_dataset, register_dataset  # noqa: F401
from .scoring import SCORERS, rouge, exact_match, register_scorer  # noqa: F401
from .runner import EvalRunner, LocalBackend, ServerBackend  # noqa: F401
