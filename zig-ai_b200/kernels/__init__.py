"""CUDA kernels for sm_100a: `build` compiles and loads the libraries under csrc/, `ops` exposes
them as functions on torch tensors."""
from . import build  # noqa: F401
