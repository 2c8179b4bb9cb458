"""Reading and writing safetensors files by tensor name, without a library.

Format (as the reference parses it by hand, src/quanta/minimax/loader.py:108-134): 8 bytes
little-endian header length n, n bytes of JSON ``{name: {dtype, shape, data_offsets}}`` (an optional
``__metadata__`` entry is dropped), then the tensor bytes; offsets are relative to byte 8+n.
A folder may hold one ``model.safetensors`` or shards named by ``model.safetensors.index.json``'s
``weight_map`` (loader.py:96-97).
"""

from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path

import torch

_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32,
           "I64": torch.int64, "U8": torch.uint8, "F64": torch.float64, "BOOL": torch.bool, "I8": torch.int8,
           "I16": torch.int16}
_NAMES = {v: k for k, v in _DTYPES.items()}
_QUANTIZED = ("F8_E4M3", "F8_E5M2", "F4", "F6_E2M3", "F6_E3M2", "F8_E8M0")


class SafetensorsFile:
    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._mm) < 8:
            raise ValueError(f"{self.path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", self._mm[:8])
        if 8 + n > len(self._mm):
            raise ValueError(f"{self.path}: header length {n} exceeds the file")
        self.header = json.loads(self._mm[8:8 + n])
        self.header.pop("__metadata__", None)
        self.base = 8 + n

    def names(self):
        return self.header.keys()

    def meta(self, name: str) -> tuple[str, tuple[int, ...]]:
        m = self.header[name]
        return m["dtype"], tuple(m["shape"])

    def read(self, name: str) -> torch.Tensor:
        m = self.header[name]
        dt = m["dtype"]
        if dt in _QUANTIZED:
            raise ValueError(f"{name}: stored as {dt}; quantized checkpoints are not supported")
        if dt not in _DTYPES:
            raise ValueError(f"{name}: unknown safetensors dtype {dt}")
        b, e = m["data_offsets"]
        shape = tuple(m["shape"])
        numel = 1
        for s in shape:
            numel *= s
        tdt = _DTYPES[dt]
        if e - b != numel * tdt.itemsize:
            raise ValueError(f"{name}: {e - b} bytes stored, shape {shape} of {dt} needs {numel * tdt.itemsize}")
        if numel == 0:
            return torch.empty(shape, dtype=tdt)
        buf = memoryview(self._mm)[self.base + b:self.base + e]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)     # the mapping is read-only; nothing writes to it
            return torch.frombuffer(buf, dtype=tdt).reshape(shape)

    def close(self):
        try:
            self._mm.close()
        except BufferError:      # views of the mapping are still alive; the OS unmaps at exit
            pass
        self._f.close()


def write_safetensors(path, tensors: dict[str, torch.Tensor]) -> None:
    """Write CPU tensors by name, in the given order."""
    header = {}
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise ValueError(f"{name}: dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)


class CheckpointFolder:
    """All tensors of a model folder by name (single file or sharded with an index)."""

    def __init__(self, model_dir):
        d = Path(model_dir)
        self.dir = d
        self._files: dict[str, SafetensorsFile] = {}
        self._where: dict[str, str] = {}
        index = d / "model.safetensors.index.json"
        if index.exists():
            wm = json.loads(index.read_text()).get("weight_map")
            if not isinstance(wm, dict) or not wm:
                raise ValueError(f"{index}: no weight_map")
            shards = sorted(set(wm.values()))
            absent = [fn for fn in shards if not (d / fn).is_file()]
            if absent:
                raise FileNotFoundError(f"{index.name} names {len(absent)} shard(s) that are not in {d}: "
                                        f"{', '.join(absent[:8])}")
            for fn in shards:
                self._files[fn] = SafetensorsFile(d / fn)
            astray = sorted(name for name, fn in wm.items() if name not in self._files[fn].header)
            if astray:
                raise ValueError(f"{index.name} places {len(astray)} tensor(s) in shards that do not hold them: "
                                 f"{', '.join(astray[:8])}")
            self._where.update(wm)
        else:
            single = d / "model.safetensors"
            files = [single] if single.exists() else sorted(d.glob("*.safetensors"))
            if not files:
                raise FileNotFoundError(f"{d}: no model.safetensors (or index, or *.safetensors) found")
            for p in files:
                sf = SafetensorsFile(p)
                self._files[p.name] = sf
                for name in sf.names():
                    self._where[name] = p.name

    def names(self) -> list[str]:
        return list(self._where)

    def meta(self, name: str):
        return self._files[self._where[name]].meta(name)

    def read(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].read(name)

    def close(self):
        for f in self._files.values():
            f.close()
