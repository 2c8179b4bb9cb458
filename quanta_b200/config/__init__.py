"""Typed configurations and the architecture registry."""
from .minimax_m3 import ConfigError, MiniMaxM3Config  # noqa: F401
from .registry import known_architectures, load_config, register_architecture, resolve  # noqa: F401
