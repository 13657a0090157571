"""Reading and writing the safetensors container.

Layout (as the reference parses it, src/model/model_loader.cpp:41-103): an
8-byte little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` with offsets relative to
the end of the header, then the raw little-endian data.  ``__metadata__`` is
skipped.  Unlike the reference, which turns every tensor into host fp32 and
checks neither byte counts nor dtypes it does not know, the file is mapped, each
entry's byte count is checked against shape x element size, and an unknown dtype
is an error.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

# safetensors dtype -> (bytes per element, numpy dtype used to view the bytes, torch dtype)
_DTYPES = {
    "F32": (4, np.float32, torch.float32),
    "F16": (2, np.float16, torch.float16),
    "BF16": (2, np.uint16, torch.bfloat16),
    "F64": (8, np.float64, torch.float64),
    "I64": (8, np.int64, torch.int64),
    "I32": (4, np.int32, torch.int32),
    "I16": (2, np.int16, torch.int16),
    "I8": (1, np.int8, torch.int8),
    "U8": (1, np.uint8, torch.uint8),
    "BOOL": (1, np.uint8, torch.bool),
}
_TORCH_TO_ST = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                torch.float64: "F64", torch.int64: "I64", torch.int32: "I32",
                torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A mapped safetensors file; ``tensor(name)`` returns a CPU tensor viewing the map."""

    def __init__(self, path: str):
        self.path = path
        if not os.path.isfile(path):
            raise SafetensorsError(f"weights file not found: {path}")
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header ({size} bytes)")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape, (b, en) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for tensor {name!r}") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype!r}")
            numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if en - b != numel * _DTYPES[dtype][0]:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} of shape {list(shape)} and dtype {dtype} needs "
                    f"{numel * _DTYPES[dtype][0]} bytes, header gives {en - b}")
            if b < 0 or en > data_len:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} lies at bytes [{b}, {en}) beyond the data section of {data_len} bytes "
                    "(truncated file?)")
            self.entries[name] = (dtype, shape, b, en)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> str:
        return self.entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, b, e = self.entries[name]
        _, np_dt, th_dt = _DTYPES[dtype]
        arr = np.frombuffer(self._map, dtype=np_dt, count=(e - b) // np.dtype(np_dt).itemsize,
                            offset=self._data_start + b)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")       # the map is read-only; the tensor is only read
            t = torch.from_numpy(arr.copy() if arr.size == 0 else arr)
        if dtype == "BF16":
            t = t.view(torch.bfloat16)
        elif dtype == "BOOL":
            t = t.to(torch.bool)
        return t.reshape(shape)

    def close(self):
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:      # a tensor still views the map; it goes with the last view
                pass
            self._map = None
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write ``tensors`` (CPU or device) to ``path``; data starts 8-byte aligned."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_ST:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            elif t.dtype == torch.bool:
                t = t.to(torch.uint8)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)
