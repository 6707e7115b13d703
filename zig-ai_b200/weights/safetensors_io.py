"""Reading and writing the safetensors container.

Layout: an 8-byte little-endian header length, a JSON header that maps each tensor name to its
dtype, shape and `data_offsets` [begin, end), then the data; offsets count from the first byte
after the header, so a tensor starts at file offset `8 + header_len + begin`.  (The reference's
header parser, src/loader/safetensors.zig:59-246, documents the same layout at :1-15 and :87-105
but leaves the header length out of the data offset at :225-229.)
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Tuple

import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """The header of one file; tensors are read one at a time by name."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise SafetensorsError(f"{path}: too short for a safetensors header")
            (n,) = struct.unpack("<Q", head)
            if n < 2 or 8 + n > size:
                raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
            try:
                header = json.loads(f.read(n).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header should be a JSON object")
        self.data_start = 8 + n
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                dtype, shape, (b, en) = e["dtype"], tuple(int(x) for x in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError) as err:
                raise SafetensorsError(f"{path}: malformed entry for '{name}'") from err
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype}")
            count = 1
            for x in shape:
                count *= x
            if en - b != count * _DTYPES[dtype][1] or b < 0 or self.data_start + en > size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' ({dtype}{list(shape)}) does not match its data offsets [{b}, {en}) "
                    f"or runs past the end of the file")
            self.entries[name] = (dtype, shape, b, en)

    def names(self):
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self.entries[name]
        return _DTYPES[dtype][0], shape

    def read(self, name: str) -> torch.Tensor:
        dtype, shape, b, en = self.entries[name]
        buf = bytearray(en - b)
        with open(self.path, "rb") as f:
            f.seek(self.data_start + b)
            got = f.readinto(buf)
        if got != en - b:
            raise SafetensorsError(f"{self.path}: short read for '{name}'")
        if en == b:
            return torch.empty(shape, dtype=_DTYPES[dtype][0])
        return torch.frombuffer(buf, dtype=_DTYPES[dtype][0]).reshape(shape)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of '{name}'")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
