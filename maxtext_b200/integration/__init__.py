"""Bridges to external serving / RL stacks (src/maxtext/integration/)."""
