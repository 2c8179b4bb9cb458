"""Architectures: each module maps a configuration to a model specification and registers itself."""
from . import minimax_m3  # noqa: F401
