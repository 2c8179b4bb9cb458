"""quanta_b200: a small, whole inference engine for one B200 (sm_100a), one model architecture at a
time, from a model folder (config.json + safetensors) to tokens.

Public entry points: ``generate`` (programmatic), ``python -m quanta_b200 generate`` (command line),
``bin/trace_run`` (replay of given token ids, logits out).
"""

from .config.registry import known_architectures, load_config, register_architecture  # noqa: F401

__all__ = ["generate", "load_model", "Engine", "known_architectures", "load_config", "register_architecture"]


def __getattr__(name):
    # torch-heavy modules are imported on first use, so configuration tools stay light
    if name == "generate":
        from .engine.generate import generate
        return generate
    if name == "load_model":
        from .engine.model import load_model
        return load_model
    if name == "Engine":
        from .engine.step import Engine
        return Engine
    raise AttributeError(name)
