"""Reading and writing the safetensors container, by tensor name.

The format: 8 bytes little-endian header length, a JSON header mapping each
tensor name to {"dtype", "shape", "data_offsets": [begin, end]} (offsets count
from the end of the header), then the raw little-endian data.  The reference
binds tensors by name out of a memory-mapped GGUF file in the same spirit
(src/lfm25_model.c:35-49, src/gguf_parser.c:58-84); this engine's checkpoints
are safetensors.  A folder may hold one `model.safetensors` or shards listed in
`model.safetensors.index.json`.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_CODES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    file: str
    begin: int          # absolute byte offset in the file
    nbytes: int


class SafetensorsFile:
    """One memory-mapped .safetensors file."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > size - 8 or hlen > (1 << 30):
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        base = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            code = info.get("dtype")
            if code not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {code!r}")
            dt, width = _DTYPES[code]
            shape = tuple(int(s) for s in info["shape"])
            b, e = (int(v) for v in info["data_offsets"])
            want = int(np.prod(shape, dtype=np.int64)) * width if shape else width
            if e - b != want or base + e > size or b < 0:
                raise SafetensorsError(f"{path}: tensor {name!r} claims bytes [{b},{e}) for shape {list(shape)} "
                                       f"{code}, which needs {want} bytes in a file of {size}")
            self.entries[name] = TensorEntry(name, dt, shape, path, base + b, e - b)
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def tensor(self, name: str) -> torch.Tensor:
        """A host tensor that copies the named tensor's bytes out of the mapping."""
        e = self.entries[name]
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=e.nbytes, offset=e.begin)
        t = torch.from_numpy(buf.copy())
        return t.view(e.dtype).reshape(e.shape) if e.nbytes else torch.empty(e.shape, dtype=e.dtype)

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._fh.close()


class ModelFiles:
    """All tensors of a model folder, whichever shard holds them."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        names: list[str]
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                wm = json.load(f).get("weight_map", {})
            names = sorted(set(wm.values()))
        elif os.path.isfile(single):
            names = ["model.safetensors"]
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")
        self.files = [SafetensorsFile(os.path.join(model_dir, n)) for n in names]
        self.entries: Dict[str, TensorEntry] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        for sf in self.files:
            for n, e in sf.entries.items():
                if n in self.entries:
                    raise SafetensorsError(f"{model_dir}: tensor {n!r} appears in more than one shard")
                self.entries[n] = e
                self._owner[n] = sf

    def tensor(self, name: str) -> torch.Tensor:
        return self._owner[name].tensor(name)

    def close(self) -> None:
        for sf in self.files:
            sf.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] | None = None) -> None:
    """Writes (name, tensor) pairs in the given order; data blocks are 8-byte aligned."""
    items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for n, t in items:
        if t.dtype not in _CODES:
            raise SafetensorsError(f"tensor {n!r}: dtype {t.dtype} cannot be written")
        nbytes = t.numel() * t.element_size()
        header[n] = {"dtype": _CODES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
