from .diloco import DiLoCoTrainer, fragments_of, nesterov_outer_step, streaming_schedule  # noqa: F401
