"""Weights by tensor name: sources, the check against what the parts expect, and the fetch.

The parts of a model name every tensor they need with its shape (``TensorSpec``).  ``open_fetch``
compares that list with what a source holds and raises ONE ``WeightError`` listing missing and
unexpected tensors and wrong shapes (the reference checks coverage both ways,
src/quanta/minimax/quant_policy_m3.py:98-121, and names a missing key, loader.py:121-122).  Matrices
are held in the compute dtype (bfloat16 for serving; float32 for the true 32-bit path); tensors of
kind ``f32`` (norm gains, router gate and bias) are float32 in both.
"""

from __future__ import annotations

import hashlib
from typing import Callable, Iterable

import torch

from ..parts.base import TensorSpec
from .safetensors_io import CheckpointFolder

_ST_NAME = {torch.float32: "F32", torch.bfloat16: "BF16", torch.int32: "I32"}


class WeightError(ValueError):
    pass


class FolderSource:
    """Tensors of a model folder (config.json beside model.safetensors or shards)."""

    def __init__(self, model_dir):
        self.ckpt = CheckpointFolder(model_dir)

    def names(self) -> list[str]:
        return self.ckpt.names()

    def meta(self, name: str):
        return self.ckpt.meta(name)

    def read(self, name: str, device) -> torch.Tensor:
        return self.ckpt.read(name)

    def close(self):
        self.ckpt.close()


class DictSource:
    """Tensors handed over in memory, by name."""

    def __init__(self, tensors: dict):
        self.tensors = dict(tensors)

    def names(self) -> list[str]:
        return list(self.tensors)

    def meta(self, name: str):
        t = self.tensors[name]
        return _ST_NAME.get(t.dtype, str(t.dtype)), tuple(t.shape)

    def read(self, name: str, device) -> torch.Tensor:
        return self.tensors[name]

    def close(self):
        pass


def _seed_for(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & (2 ** 63 - 1)


class RandomSource:
    """Seeded random tensors for a list of specs; a tensor depends on (seed, its name) and on the kind of
    device it is drawn on (the CPU's and the GPU's generators differ, and large matrices are drawn in
    bfloat16 directly on the GPU), so the order of generation does not matter, and the same seed on the same
    kind of device gives the same model; a folder written by the random-weights mode (drawn on the CPU) and a
    model drawn on the GPU from the same seed are two different models.  ``normal``: N(0, 0.02); ``gain``: 1 + U(-0.1, 0.1); ``bias``:
    U(-0.05, 0.05).  Matrices are drawn in float32 and rounded to ``matrix_dtype``."""

    def __init__(self, specs: Iterable[TensorSpec], seed: int, matrix_dtype=torch.bfloat16):
        self.specs = {s.name: s for s in specs}
        self.seed = int(seed)
        self.matrix_dtype = matrix_dtype
        self._gens = {}

    def names(self) -> list[str]:
        return list(self.specs)

    def meta(self, name: str):
        s = self.specs[name]
        dt = self.matrix_dtype if s.kind == "matrix" else (torch.int32 if s.kind == "i32" else torch.float32)
        return _ST_NAME[dt], tuple(s.shape)

    def read(self, name: str, device="cpu") -> torch.Tensor:
        s = self.specs[name]
        device = torch.device(device)
        key = str(device)
        if key not in self._gens:
            self._gens[key] = torch.Generator(device=device)
        g = self._gens[key]
        g.manual_seed(_seed_for(self.seed, name))
        if s.init == "normal":
            big = device.type == "cuda" and s.kind == "matrix"
            t = torch.empty(s.shape, dtype=self.matrix_dtype if big else torch.float32, device=device)
            t.normal_(0.0, 0.02, generator=g)
        elif s.init == "gain":
            t = torch.empty(s.shape, dtype=torch.float32, device=device).uniform_(-0.1, 0.1, generator=g) + 1.0
        elif s.init == "bias":
            t = torch.empty(s.shape, dtype=torch.float32, device=device).uniform_(-0.05, 0.05, generator=g)
        else:
            raise ValueError(f"{name}: unknown init {s.init!r}")
        return t.to(self.matrix_dtype) if s.kind == "matrix" else t

    def close(self):
        pass


def _canonical(name: str, aliases) -> str:
    for file_prefix, spec_prefix in aliases:
        if name.startswith(file_prefix):
            return spec_prefix + name[len(file_prefix):]
    return name


def open_fetch(source, specs: list[TensorSpec], *, compute_dtype: torch.dtype, device, aliases=(),
               ignored_prefixes=(), ignorable=(), max_listed: int = 12) -> Callable[[str], torch.Tensor]:
    """Check ``source`` against ``specs``; return ``fetch(name) -> device tensor``."""
    want = {}
    for s in specs:
        if s.name in want and want[s.name].shape != s.shape:
            raise WeightError(f"two parts ask for {s.name} with shapes {want[s.name].shape} and {s.shape}")
        want[s.name] = s
    in_file: dict[str, str] = {}
    skipped = 0
    unexpected, quantized = [], []
    for fname in source.names():
        cname = _canonical(fname, aliases)
        if cname in want:
            in_file[cname] = fname
            continue
        if any(cname.startswith(p) or fname.startswith(p) for p in ignored_prefixes) or cname in ignorable:
            skipped += 1
            continue
        if cname.endswith(".weight_scale_inv") or cname.endswith(".weight_scale"):
            quantized.append(fname)
        else:
            unexpected.append(fname)
    missing = [n for n in want if n not in in_file]
    wrong = []
    for cname, fname in in_file.items():
        dt, shape = source.meta(fname)
        if dt.startswith("F8") or dt.startswith("F4") or dt.startswith("F6"):
            quantized.append(fname)
        elif tuple(shape) != tuple(want[cname].shape):
            wrong.append(f"{fname}: stored {list(shape)}, expected {list(want[cname].shape)}")
        elif dt not in ("F32", "BF16", "F16", "F64", "I32", "I64"):
            wrong.append(f"{fname}: stored dtype {dt} cannot be used")

    def some(xs):
        xs = sorted(xs)
        more = f" ... and {len(xs) - max_listed} more" if len(xs) > max_listed else ""
        return ", ".join(xs[:max_listed]) + more

    problems = []
    if missing:
        problems.append(f"{len(missing)} missing tensor(s): {some(missing)}")
    if unexpected:
        problems.append(f"{len(unexpected)} unexpected tensor(s): {some(unexpected)}")
    if wrong:
        problems.append(f"{len(wrong)} tensor(s) of the wrong shape or dtype: {some(wrong)}")
    if quantized:
        problems.append(f"{len(quantized)} quantized tensor(s) (fp8 blocks or scale grids; quantized "
                        f"checkpoints are not supported): {some(quantized)}")
    if problems:
        raise WeightError("the checkpoint does not fit the model: " + "; ".join(problems))

    def fetch(name: str) -> torch.Tensor:
        s = want[name]
        t = source.read(in_file[name], device)
        target = compute_dtype if s.kind == "matrix" else (torch.int32 if s.kind == "i32" else torch.float32)
        return t.to(device=device, dtype=target)

    fetch.skipped = skipped          # tensors of other towers that were passed over
    return fetch
