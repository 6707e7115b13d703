"""Loading a model's tensors by name from a model folder.

The reference looks tensors up by name in the GGUF file (`getTensor`, src/loader/gguf.zig:395;
per-layer prefix `blk.{i}.`, src/transformer/hybrid_layer.zig:295) and fails on the first missing
or misshapen one (`WeightFileNotFound`, `ShapeMismatch`, src/transformer/short_conv.zig:27-30).
Here every expected tensor is checked first and one error lists all that is missing, unexpected,
of the wrong shape or of an unusable dtype.

Kept dtypes: matrices and the embedding table follow the model's dtype, except that a tensor
stored in 32-bit stays 32-bit; small vectors (norm weights, conv taps, biases) are kept in 32-bit;
integer tensors become int32.  In the 32-bit mode every floating tensor is 32-bit.
"""
from __future__ import annotations

import glob
import os
from typing import Dict

import torch

from ..parts.base import ParamDecl
from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """The tensors of a model folder do not fit the model."""

    def __init__(self, where, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"{where}: the tensors do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} expected {list(want)}, file has {list(got)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  unusable dtype: {name} is stored as {got}")
        super().__init__("\n".join(lines))


_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def kept_dtype(decl: ParamDecl, stored: torch.dtype, model_dtype: torch.dtype):
    if stored in _INTS:
        return torch.int32
    if stored not in _FLOATS:
        return None
    if model_dtype == torch.float32 or decl.role == "vector" or stored in (torch.float32, torch.float64):
        return torch.float32
    return model_dtype


def open_model_files(model_dir: str):
    paths = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not paths:
        raise SafetensorsError(f"no .safetensors file in {model_dir}")
    return [SafetensorsFile(p) for p in paths]


def load_tensors(model_dir: str, decls: Dict[str, ParamDecl], model_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    files = open_model_files(model_dir)
    where_of = {}
    duplicates = []
    for f in files:
        for name in f.names():
            if name in where_of:
                duplicates.append(name)
            where_of[name] = f
    missing = [n for n in decls if n not in where_of]
    unexpected = [n for n in where_of if n not in decls] + [n + " (stored twice)" for n in duplicates]
    wrong_shape, wrong_dtype = [], []
    for name, decl in decls.items():
        if name not in where_of:
            continue
        stored, shape = where_of[name].info(name)
        if tuple(shape) != tuple(decl.shape) and tuple(shape) not in decl.alt_shapes:
            wrong_shape.append((name, decl.shape, shape))
        if kept_dtype(decl, stored, model_dtype) is None:
            wrong_dtype.append((name, str(stored)))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_dtype)
    out = {}
    for name, decl in decls.items():
        t = where_of[name].read(name)
        keep = kept_dtype(decl, t.dtype, model_dtype)
        out[name] = t.reshape(decl.shape).to(device=device, dtype=keep).contiguous()
    return out
