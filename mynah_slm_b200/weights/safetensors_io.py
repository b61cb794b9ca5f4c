"""A small safetensors reader and writer (no third-party package).

File layout as the reference's vendored reader handles it (mynah-slm
third_party/ingot/src/safetensors.c:357-403 header, :224-322 one tensor
object, :636-701 folder resolution): an 8-byte little-endian header length, a
JSON object `{name: {dtype, shape, data_offsets}}` (plus an optional
`__metadata__`), then the payload. A folder is `model.safetensors.index.json`
with its shards, or `model.safetensors`, or every `*.safetensors` in sorted
order. The malformed-file cases refused here are those of
third_party/ingot/tests/test_safetensors.c:232-297.

Tensors are handed out as zero-copy CPU views of a private file mapping.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Iterable, Mapping

import torch


class SafetensorsError(ValueError):
    """A safetensors file that cannot be trusted."""


DTYPES: dict[str, torch.dtype] = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
    "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8, "F64": torch.float64,
}
_NAMES = {v: k for k, v in DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: tuple[int, ...]
    begin: int          # offsets into the payload
    end: int
    file: "SafetensorsFile"

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: shorter than its 8-byte header length")
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header of {hlen} bytes is longer than the file")
        try:
            table = json.loads(self._fh.read(hlen))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(table, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self.payload_offset = 8 + hlen
        payload = size - self.payload_offset
        self.metadata = table.pop("__metadata__", None)
        self.entries: dict[str, TensorEntry] = {}
        for name, t in table.items():
            if not isinstance(t, dict):
                raise SafetensorsError(f"{path}: entry {name!r} is not an object")
            for k in ("dtype", "shape", "data_offsets"):
                if k not in t:
                    raise SafetensorsError(f"{path}: tensor {name!r} has no {k}")
            dt, shape, offs = t["dtype"], t["shape"], t["data_offsets"]
            if dt not in DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            if not (isinstance(shape, list) and all(isinstance(s, int) and s >= 0 for s in shape)):
                raise SafetensorsError(f"{path}: tensor {name!r} has a malformed shape {shape!r}")
            if not (isinstance(offs, list) and len(offs) == 2 and all(isinstance(o, int) for o in offs)):
                raise SafetensorsError(f"{path}: tensor {name!r} has malformed data_offsets {offs!r}")
            lo, hi = offs
            if lo > hi:
                raise SafetensorsError(f"{path}: tensor {name!r} has reversed offsets [{lo}, {hi}]")
            if hi > payload:
                raise SafetensorsError(f"{path}: tensor {name!r} ends at {hi}, past the payload of {payload} bytes")
            e = TensorEntry(name, dt, tuple(shape), lo, hi, self)
            want = e.numel * DTYPES[dt].itemsize
            if hi - lo != want:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} holds {hi - lo} bytes, its shape and dtype need {want}")
            self.entries[name] = e
        self._map = None

    def _mapping(self):
        if self._map is None:
            # a private (copy-on-write) mapping: torch wants a writable buffer
            self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY)
        return self._map

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if e.numel == 0:
            return torch.empty(e.shape, dtype=DTYPES[e.dtype])
        t = torch.frombuffer(self._mapping(), dtype=DTYPES[e.dtype], count=e.numel,
                             offset=self.payload_offset + e.begin)
        return t.reshape(e.shape)

    def close(self) -> None:
        # views handed out keep the mapping alive; only the descriptor is dropped
        self._map = None
        self._fh.close()


class Checkpoint:
    """All tensors of a model folder, whichever way it is sharded."""

    def __init__(self, folder: str):
        self.folder = folder
        self.files: list[SafetensorsFile] = []
        self.entries: dict[str, TensorEntry] = {}
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        if os.path.isfile(index):
            with open(index) as f:
                weight_map = json.load(f).get("weight_map")
            if not isinstance(weight_map, dict):
                raise SafetensorsError(f"{index}: no weight_map")
            shards = sorted(set(weight_map.values()))
            paths = [os.path.join(folder, s) for s in shards]
        elif os.path.isfile(single):
            paths = [single]
        else:
            paths = sorted(os.path.join(folder, n) for n in os.listdir(folder) if n.endswith(".safetensors"))
        if not paths:
            raise SafetensorsError(f"no safetensors file in {folder}")
        for p in paths:
            if not os.path.isfile(p):
                raise SafetensorsError(f"shard {p} named by the index does not exist")
            sf = SafetensorsFile(p)
            self.files.append(sf)
            for name, e in sf.entries.items():
                if name in self.entries:
                    raise SafetensorsError(
                        f"tensor {name!r} appears in both {self.entries[name].file.path} and {p}")
                self.entries[name] = e

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def tensor(self, name: str) -> torch.Tensor:
        return self.entries[name].file.tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Mapping[str, str] | None = None) -> None:
    """Write tensors in the given order; the header is padded with spaces so
    that the payload starts on an 8-byte boundary."""
    table: dict[str, object] = {}
    if metadata:
        table["__metadata__"] = dict(metadata)
    offset = 0
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot write {name!r}: dtype {t.dtype}")
        n = t.numel() * t.element_size()
        table[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    header = json.dumps(table, separators=(",", ":")).encode()
    header += b" " * (-(8 + len(header)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(header)))
        f.write(header)
        for name, t in tensors.items():
            c = t.detach().cpu().contiguous()
            if c.numel():
                f.write(c.reshape(-1).view(torch.uint8).numpy())
    os.replace(tmp, path)
