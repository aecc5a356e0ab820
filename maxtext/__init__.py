"""Compatibility import path: `python -m maxtext.train ...` and the reference's module names resolve to
`maxtext_b200`."""
from maxtext_b200 import __version__  # noqa: F401
