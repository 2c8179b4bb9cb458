"""A model built from a specification: parts instantiated, weights loaded, layers run in schedule order.

The model owns no cache and no request state; the step function hands it the step's context, the
per-entry cache views and state rows.  It runs exactly the tokens it is given and returns float32
logits at the wanted rows.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from .. import matmul
from ..config.registry import load_config
from ..parts import block as _block  # noqa: F401  (registers the built-in block, embedding and head)
from ..parts.base import CacheSpec, Part, TensorSpec, make
from ..parts.spec import ModelSpec
from ..weights.loader import FolderSource, RandomSource, open_fetch
from ..weights.safetensors_io import write_safetensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(d) -> torch.dtype:
    try:
        return _DTYPES[d]
    except KeyError:
        raise ValueError(f"dtype {d!r}: choose bfloat16 or float32") from None


def _walk(part: Part):
    yield part
    for c in part.children():
        yield from _walk(c)


class Model:
    def __init__(self, spec: ModelSpec, dtype=torch.bfloat16, device="cuda:0"):
        self.spec = spec
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        self.embedding = make("embedding", spec.embedding)
        self.blocks = [make("block", choice) for choice in spec.layers]
        self.head = make("head", spec.head)
        self.schedule = list(spec.schedule)
        self.loaded = False

    # ---- weights -------------------------------------------------------------------------------
    def parts(self):
        for top in [self.embedding, *self.blocks, self.head]:
            yield from _walk(top)

    def tensor_specs(self) -> list[TensorSpec]:
        out, seen = [], set()
        for p in self.parts():
            for s in p.tensor_specs():
                if s.name not in seen:
                    seen.add(s.name)
                    out.append(s)
        return out

    def load(self, source) -> "Model":
        ignorable = ("lm_head.weight",) if self.spec.tied_head else ()
        fetch = open_fetch(source, self.tensor_specs(), compute_dtype=self.dtype, device=self.device,
                           aliases=self.spec.name_aliases, ignored_prefixes=self.spec.ignored_prefixes,
                           ignorable=ignorable)
        # a tensor that several parts ask for by the same name (a head tied to the embedding table) is
        # loaded once and shared
        shared: dict[str, torch.Tensor] = {}
        asked: dict[str, int] = {}
        for p in self.parts():
            for ts in p.tensor_specs():
                asked[ts.name] = asked.get(ts.name, 0) + 1
        share = {name for name, n in asked.items() if n > 1}

        def fetch_shared(name):
            if name in share:
                if name not in shared:
                    shared[name] = fetch(name)
                return shared[name]
            return fetch(name)

        for p in self.parts():
            p.load(fetch_shared)
        self.loaded = True
        return self

    # ---- what the cache manager needs to know ---------------------------------------------------
    def cache_needs(self) -> list[CacheSpec | None]:
        """For each schedule position that writes a cache, the mixer's need (None: the mixer keeps none)."""
        return [None if e.read_cache_of is not None else self.blocks[e.layer].mixer.cache_spec()
                for e in self.schedule]

    def state_needs(self) -> list[dict]:
        return [self.blocks[e.layer].mixer.state_spec() for e in self.schedule]

    # ---- one step --------------------------------------------------------------------------------
    def forward(self, token_ids, ctx, caches, states, want_rows):
        """``token_ids`` int32 [T]; ``caches[pos]``/``states[pos]`` per schedule position; ``want_rows``
        int32 rows whose logits are returned ([n, vocab] float32) or None."""
        h = self.embedding.forward(token_ids, ctx)
        pending = None
        for pos, entry in enumerate(self.schedule):
            pending = self.blocks[entry.layer].forward(h, pending, ctx, caches[pos], states[pos])
        if want_rows is None or want_rows.numel() == 0:
            return None
        return self.head.forward(h, pending, want_rows, ctx)


# ------------------------------------------------------------------------------------------------
def load_model(model_dir, dtype="bfloat16", device="cuda:0") -> tuple[Model, object]:
    """Model folder (config.json + safetensors) -> (loaded model, its configuration)."""
    from .. import models  # noqa: F401  (registers the architectures)
    matmul.configure()
    arch, cfg = load_config(model_dir)
    model = Model(arch.build_spec(cfg), dtype=dtype, device=device)
    src = FolderSource(model_dir)
    try:
        model.load(src)
    finally:
        src.close()
    return model, cfg


def random_model(cfg, seed: int, dtype="bfloat16", device="cuda:0", arch=None) -> Model:
    """Seeded random weights generated on the device, no files (for sizes too large to write)."""
    from .. import models  # noqa: F401
    from ..config.registry import resolve
    matmul.configure()
    arch = arch or resolve(cfg.to_dict())
    model = Model(arch.build_spec(cfg), dtype=dtype, device=device)
    model.load(RandomSource(model.tensor_specs(), seed, matrix_dtype=torch.bfloat16))
    return model


def write_random_model(cfg, seed: int, out_dir, matrix_dtype=torch.bfloat16) -> Path:
    """Random-weights mode: write ``config.json`` and ``model.safetensors`` from a configuration and a seed."""
    from .. import models  # noqa: F401
    from ..config.registry import resolve
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    raw = cfg.to_dict()
    arch = resolve(raw)
    model = Model(arch.build_spec(cfg), dtype=torch.float32, device="cpu")
    specs = model.tensor_specs()
    src = RandomSource(specs, seed, matrix_dtype=matrix_dtype)
    tensors = {s.name: src.read(s.name, "cpu") for s in specs}
    write_safetensors(out / "model.safetensors", tensors)
    (out / "config.json").write_text(json.dumps(raw, indent=1))
    return out
