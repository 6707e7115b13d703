"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has random tensors only in tests and benchmarks (`Tensor.randUniform` / `randn`
over Xoshiro256, src/tensor.zig:241-258).  Distributions: matrices and the embedding N(0, 0.02^2),
norm weights 1 + U(-0.1, 0.1), convolution taps and biases N(0, 0.1^2).  Each tensor has its own
generator seeded from the seed and the tensor's name, so a tensor's values do not depend on which
other tensors the model has.
"""
from __future__ import annotations

import os
import zlib
from typing import Dict

import torch

from ..config.base import ModelConfig, save_config
from ..parts.base import ParamDecl
from .safetensors_io import write_safetensors


def random_tensor(name: str, decl: ParamDecl, seed: int, store_dtype: torch.dtype,
                  matrix_std="fixed") -> torch.Tensor:
    """`matrix_std`: "fixed" gives matrices the standard deviation 0.02; "fan_in" gives a matrix
    [out, in] the deviation 1/sqrt(in), which keeps every part's output near unit size (used by
    tests, where a part that contributes nothing would hide its faults)."""
    g = torch.Generator(device="cpu")
    g.manual_seed((int(seed) * 0x9E3779B1 + zlib.crc32(name.encode("utf-8"))) % (2 ** 63))
    if decl.init == "norm_weight":
        t = 1.0 + (torch.rand(decl.shape, generator=g, dtype=torch.float32) * 0.2 - 0.1)
    elif decl.init == "conv":
        t = torch.randn(decl.shape, generator=g, dtype=torch.float32) * 0.1
    else:
        std = 0.02
        if matrix_std == "fan_in" and decl.role == "matrix" and len(decl.shape) == 2:
            std = float(decl.shape[1]) ** -0.5
        elif matrix_std not in ("fixed", "fan_in"):
            raise ValueError(f"matrix_std should be 'fixed' or 'fan_in', got {matrix_std!r}")
        t = torch.randn(decl.shape, generator=g, dtype=torch.float32) * std
    return t.to(store_dtype)


def random_tensors(decls: Dict[str, ParamDecl], seed: int, store_dtype: torch.dtype = torch.bfloat16,
                   matrix_std="fixed"):
    return {name: random_tensor(name, decl, seed, store_dtype, matrix_std) for name, decl in decls.items()}


def write_random_model(cfg: ModelConfig, seed: int, model_dir: str, store_dtype: torch.dtype = torch.bfloat16,
                       matrix_std="fixed") -> str:
    """Create `model_dir` with config.json and model.safetensors for `cfg`."""
    from ..models import build_model
    model = build_model(cfg)
    os.makedirs(model_dir, exist_ok=True)
    save_config(cfg, model_dir)
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      random_tensors(model.param_decls(), seed, store_dtype, matrix_std),
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
