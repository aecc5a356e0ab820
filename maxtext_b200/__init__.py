"""maxtext_b200: a Blackwell-native LLM training / inference library with MaxText's configuration
surface, model zoo, sharding rules and checkpoint layout, built on PyTorch, hand-written sm_100a
CUDA kernels and NCCL / NVLink symmetric memory."""
__version__ = "0.1.0"
