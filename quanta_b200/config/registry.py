"""One registry from an architecture's name to its configuration class and model builder.

A model folder's ``config.json`` names its architecture in ``architectures[0]`` and/or
``model_type``; ``resolve`` looks both up here (the reference dispatches on ``model_type`` with a
most-specific-first prefix chain, src/quanta/shim/omlx.py:307-341, and raises on an unknown one).

Adding an architecture is one call to ``register_architecture`` from the module that defines its
configuration and its ``build_spec`` function; nothing else in the framework names a model.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Any                     # has from_dict(raw, generation=None)
    build_spec: Callable[[Any], Any]    # config -> parts.spec.ModelSpec


_BY_NAME: dict[str, Architecture] = {}


def register_architecture(names, config_cls, build_spec) -> Architecture:
    names = [names] if isinstance(names, str) else list(names)
    arch = Architecture(names[0], config_cls, build_spec)
    for n in names:
        _BY_NAME[n] = arch
    return arch


def _load_builtin() -> None:
    from .. import models  # noqa: F401  (each architecture module registers itself on import)


def known_architectures() -> list[str]:
    _load_builtin()
    return sorted(_BY_NAME)


def resolve(raw_config: dict) -> Architecture:
    """Architecture for a raw ``config.json`` dictionary; unknown names raise with the known list."""
    _load_builtin()
    candidates = list(raw_config.get("architectures") or [])
    if raw_config.get("model_type"):
        candidates.append(str(raw_config["model_type"]))
    tc = raw_config.get("text_config") or {}
    if tc.get("model_type"):
        candidates.append(str(tc["model_type"]))
    for c in candidates:
        if c in _BY_NAME:
            return _BY_NAME[c]
    raise KeyError(f"no registered architecture among {candidates or '(config.json names none)'}; "
                   f"known: {known_architectures()}")


def load_config(model_dir) -> tuple[Architecture, Any]:
    """Read ``config.json`` (and ``generation_config.json`` if present) of a model folder."""
    d = Path(model_dir)
    path = d / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"{path} not found: a model folder holds config.json and model.safetensors")
    raw = json.loads(path.read_text())
    gen = None
    gp = d / "generation_config.json"
    if gp.exists():
        gen = json.loads(gp.read_text())
    arch = resolve(raw)
    return arch, arch.config_cls.from_dict(raw, generation=gen)
