"""Reader and writer for the safetensors container.

Format (as the reference parses it, src/core/safetensors.cpp:28-71): an 8-byte
little-endian header length, a JSON header ``{name: {dtype, shape,
data_offsets:[begin,end]}}`` (``__metadata__`` skipped), then the raw tensor
bytes; offsets are relative to the end of the header.  A folder may hold one
``model.safetensors`` or a ``model.safetensors.index.json`` whose ``weight_map``
names shard files (safetensors.cpp:75-104).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    path: str
    begin: int  # absolute byte offset in the file
    nbytes: int


def read_header(path: str) -> Dict[str, TensorEntry]:
    try:
        size = os.path.getsize(path)
        f = open(path, "rb")
    except OSError as e:
        raise SafetensorsError(f"cannot open {path!r}: {e}") from e
    with f:
        if size < 8:
            raise SafetensorsError(f"{path!r}: file shorter than the 8-byte header length")
        (hlen,) = struct.unpack("<Q", f.read(8))
        if hlen == 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path!r}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path!r}: header is not valid JSON: {e}") from e
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path!r}: header must be a JSON object")
    base = 8 + hlen
    out: Dict[str, TensorEntry] = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dt = info["dtype"]
            shape = tuple(int(s) for s in info["shape"])
            b, e = (int(x) for x in info["data_offsets"])
        except (KeyError, TypeError, ValueError) as err:
            raise SafetensorsError(f"{path!r}: malformed entry for tensor {name!r}") from err
        if dt not in _DTYPES:
            raise SafetensorsError(f"{path!r}: tensor {name!r} has unsupported dtype {dt!r}")
        tdt, isz = _DTYPES[dt]
        numel = 1
        for s in shape:
            numel *= s
        if b < 0 or e < b or base + e > size or e - b != numel * isz:
            raise SafetensorsError(
                f"{path!r}: tensor {name!r} has bad data_offsets [{b}, {e}) for shape {shape} {dt}")
        out[name] = TensorEntry(name, tdt, shape, path, base + b, e - b)
    return out


def index_folder(model_dir: str) -> Dict[str, TensorEntry]:
    """Headers of every tensor of a model folder, by name."""
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(idx):
        with open(idx, "r", encoding="utf-8") as f:
            try:
                j = json.load(f)
            except json.JSONDecodeError as e:
                raise SafetensorsError(f"{idx!r}: not valid JSON: {e}") from e
        wm = j.get("weight_map") if isinstance(j, dict) else None
        if not isinstance(wm, dict) or not wm:
            raise SafetensorsError(f"{idx!r}: missing 'weight_map'")
        entries: Dict[str, TensorEntry] = {}
        for shard in sorted(set(wm.values())):
            for name, ent in read_header(os.path.join(model_dir, shard)).items():
                if name in entries:
                    raise SafetensorsError(f"tensor {name!r} appears in more than one shard")
                entries[name] = ent
        return entries
    if os.path.isfile(single):
        return read_header(single)
    raise SafetensorsError(f"{model_dir!r} holds neither model.safetensors nor model.safetensors.index.json")


class TensorFiles:
    """Memory-maps the files of a set of entries and hands out CPU tensors (copies)."""

    def __init__(self):
        self._maps: Dict[str, Tuple[object, mmap.mmap]] = {}

    def read(self, ent: TensorEntry) -> torch.Tensor:
        if ent.path not in self._maps:
            f = open(ent.path, "rb")
            self._maps[ent.path] = (f, mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ))
        mm = self._maps[ent.path][1]
        if ent.nbytes == 0:
            return torch.empty(ent.shape, dtype=ent.dtype)
        if ent.begin + ent.nbytes > len(mm):
            raise SafetensorsError(f"{ent.path!r}: short read for tensor {ent.name!r}")
        out = torch.empty(ent.nbytes, dtype=torch.uint8)   # one copy, straight from the mapped pages
        out.numpy()[:] = np.frombuffer(mm, dtype=np.uint8, count=ent.nbytes, offset=ent.begin)
        return out.view(ent.dtype).reshape(ent.shape)

    def close(self):
        for f, mm in self._maps.values():
            mm.close()
            f.close()
        self._maps.clear()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def write_file(path: str, tensors: Mapping[str, torch.Tensor],
               metadata: Mapping[str, str] | None = None) -> None:
    """Writes ``tensors`` (CPU, any supported dtype) as one safetensors file."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    order: Iterable[str] = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
