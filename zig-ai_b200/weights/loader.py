"""Loading a model's tensors by name from a model folder.

The reference looks tensors up by name in the GGUF file (`getTensor`, src/loader/gguf.zig:395;
per-layer prefix `blk.{i}.`, src/transformer/hybrid_layer.zig:295) and fails on the first missing
or misshapen one (`WeightFileNotFound`, `ShapeMismatch`, src/transformer/short_conv.zig:27-30).
Here every expected tensor is checked first and one error lists all that is missing, unexpected,
of the wrong shape or of an unusable dtype.  Stored names go through the rename table of `names.py`
first, so a folder that spells a tensor in one of the other ways the reference accepts loads as well.
Tensors that the model does not ask for are part of that error by default; with
`unexpected="warn"` they are passed over and reported in `LoadReport.unused` instead.

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
from . import names
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


class LoadReport(dict):
    """The tensors by canonical name, with what the loader passed over: `unused` (stored, not asked
    for) and `renamed` (canonical name -> the name it was stored under, where they differ)."""
    unused: list
    renamed: dict


def load_tensors(model_dir: str, decls: Dict[str, ParamDecl], model_dtype: torch.dtype, device,
                 unexpected: str = "error") -> Dict[str, torch.Tensor]:
    files = open_model_files(model_dir)
    where_of, stored_names = {}, []
    for f in files:
        for name in f.names():
            stored_names.append(name)
            where_of.setdefault(name, f)
    by_canonical, twice, passed = names.resolve(stored_names)
    missing = [n for n in decls if n not in by_canonical]
    unused = [by_canonical[n] if by_canonical[n] == n else f"{by_canonical[n]} (= {n})" for n in by_canonical if n not in decls]
    not_wanted = (unused if unexpected == "error" else []) + [n + " (stored twice)" for n in twice]
    wrong_shape, wrong_dtype = [], []
    for name, decl in decls.items():
        if name not in by_canonical:
            continue
        stored_as = by_canonical[name]
        stored, shape = where_of[stored_as].info(stored_as)
        if tuple(shape) != tuple(decl.shape) and tuple(shape) not in decl.alt_shapes:
            wrong_shape.append((name, decl.shape, shape))
        if kept_dtype(decl, stored, model_dtype) is None:
            wrong_dtype.append((name, str(stored)))
    if missing or not_wanted or wrong_shape or wrong_dtype:
        raise WeightError(model_dir, missing, not_wanted, wrong_shape, wrong_dtype)
    out = LoadReport()
    out.unused = unused + passed
    out.renamed = {n: by_canonical[n] for n in decls if by_canonical[n] != n}
    if out.unused:
        import sys
        print(f"[zig-ai_b200] {model_dir}: {len(out.unused)} stored tensor(s) not used: " + ", ".join(out.unused[:12])
              + (" ..." if len(out.unused) > 12 else ""), file=sys.stderr)
    for name, decl in decls.items():
        stored_as = by_canonical[name]
        t = where_of[stored_as].read(stored_as)
        keep = kept_dtype(decl, t.dtype, model_dtype)
        out[name] = t.reshape(decl.shape).to(device=device, dtype=keep).contiguous()
    return out
