"""Reading and writing the safetensors container: an 8-byte little-endian header
length, a JSON header {name: {dtype, shape, data_offsets}}, then raw tensor bytes.

This takes the place of maeddesg/ROCmForge's GGUF reader (src/loader/parse.rs:28-129,
src/loader/file.rs:19-122): the file is memory-mapped and tensors are views into the
map until they are copied to the device.  Several shards are joined through
``model.safetensors.index.json``.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import torch


class SafetensorsError(IOError):
    pass


_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I32": (torch.int32, 4), "I64": (torch.int64, 8),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    file: str
    begin: int          # absolute byte offsets in the file
    end: int


class SafetensorsFile:
    """One memory-mapped .safetensors file."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        base = 8 + hlen
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
            dtype, isz = _DTYPES[info["dtype"]]
            shape = tuple(int(s) for s in info["shape"])
            b, e = info["data_offsets"]
            n = 1
            for s in shape:
                n *= s
            if e - b != n * isz:
                raise SafetensorsError(
                    f"{path}: tensor {name}: {e - b} bytes stored, shape {shape} of {info['dtype']} needs {n * isz}")
            if base + e > size:
                # src/loader/file.rs:97-103 — data must lie inside the file
                raise SafetensorsError(f"{path}: tensor {name} ends at byte {base + e}, file has {size}")
            self.entries[name] = TensorEntry(name, dtype, shape, path, base + b, base + e)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the map (read-only: copy before writing)."""
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        n = 1
        for s in e.shape:
            n *= s
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # the map is read-only by design
            t = torch.frombuffer(self._map, dtype=e.dtype, count=n, offset=e.begin)
        return t.view(e.shape)

    def close(self):
        # views handed out keep the map alive through the buffer protocol
        try:
            self._f.close()
        except Exception:
            pass


class ModelFiles:
    """All tensors of a model folder, whichever shard holds them."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        self.files: Dict[str, SafetensorsFile] = {}
        self.entries: Dict[str, TensorEntry] = {}
        if os.path.exists(index):
            with open(index) as f:
                weight_map = json.load(f).get("weight_map", {})
            shards = sorted(set(weight_map.values()))
        elif os.path.exists(single):
            shards = ["model.safetensors"]
        else:
            raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")
        for shard in shards:
            sf = SafetensorsFile(os.path.join(folder, shard))
            self.files[shard] = sf
            for name, e in sf.entries.items():
                if name in self.entries:
                    raise SafetensorsError(f"tensor {name} is stored in both {self.entries[name].file} and {e.file}")
                self.entries[name] = e
        if os.path.exists(index):
            # an index that names a tensor its shard does not hold is a stale index: say which shard
            stale = sorted(f"{name} (index says {shard})" for name, shard in weight_map.items()
                           if name not in self.files[shard].entries)
            if stale:
                raise SafetensorsError(f"{index} names tensors that their shards do not hold: " + ", ".join(stale[:8])
                                       + (f" and {len(stale) - 8} more" if len(stale) > 8 else ""))
        self._by_name = {name: sf for sf in self.files.values() for name in sf.entries}

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def tensor(self, name: str) -> torch.Tensor:
        return self._by_name[name].tensor(name)


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata=None) -> None:
    """Write (name, tensor) pairs, in the order given, as one safetensors file."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs = []
    offset = 0
    for name, t in tensors:
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
