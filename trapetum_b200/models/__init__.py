"""Architectures: each module turns a configuration into a ModelSpec and registers it."""
from . import gemma2  # noqa: F401
