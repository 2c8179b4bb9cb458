"""Weights by tensor name: safetensors reading/writing, checks, random-weights mode."""
from .loader import DictSource, FolderSource, RandomSource, WeightError, open_fetch  # noqa: F401
from .safetensors_io import CheckpointFolder, SafetensorsFile, write_safetensors  # noqa: F401
