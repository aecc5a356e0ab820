"""Block-diffusion training: tokens are noised and reconstructed block by block (src/maxtext/diffusion/block_diffusion/).

corruption        per-block random masking of a clean canvas, with the supervision masks that go with it
target_alignment  which hidden state predicts which clean token ("same_position" or "shifted")
batches           iterator wrapper that turns causal-LM batches into block-diffusion batches
"""
from .corruption import Corruption, corrupt_tokens          # noqa: F401
from .target_alignment import source_indices, align_to_targets, same_block_mask          # noqa: F401
