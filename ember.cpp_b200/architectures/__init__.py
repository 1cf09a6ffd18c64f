"""Architectures: each module turns its configuration into a ModelSpec and registers itself."""
from . import gpt2, muzozen, nipolorn  # noqa: F401
