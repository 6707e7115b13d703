"""The kernels as functions on torch CUDA tensors.

One function per kernel (or per small group launched together); every function launches on the
current CUDA stream and allocates its outputs with torch.  There is no CPU path: calling any of
these without the compiled libraries or without a CUDA device raises.  Plain matrix products go to
cuBLAS through `torch.matmul`, as the reference sends every projection to `cublasSgemm_v2`
(src/matmul/cublas.zig:515-548); the 32-bit mode runs them as true 32-bit products (TF32 off).
"""
from __future__ import annotations

import ctypes
import os
import sys
import weakref
from ctypes import c_float, c_int, c_void_p

import torch

from ..parts.base import LazyNorm
from . import build

device_type = "cuda"

_F32, _BF16 = 0, 1
_P, _I, _F = c_void_p, c_int, c_float

_SIGNATURES = {
    "embed": {
        "zai_embed": [_P, _P, _I, _P, _I, _I, _I, _P, _P],
        "zai_gather_add": [_P, _P, _P, _I, _P, _I, _I, _P],
    },
    "norm": {"zai_add_rmsnorm": [_P, _P, _P, _P, _I, _F, _I, _I, _P]},
    "activation": {"zai_silu_mul": [_P, _P, _I, _I, _I, _P]},
    "shortconv": {"zai_short_conv": [_P, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P]},
    "rope_kv": {
        "zai_rope_table": [_P, _P, _P, _I, _I, _P],
        "zai_qk_norm_rope": [_P, _I, _I, _P, _P, _F, _P, _I, _P, _P, _P, _I, _P, _I, _P, _P,
                             _I, _I, _I, _I, _I, _I, _I, _P, _P],
        "zai_kv_write": [_P, _I, _P, _I, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _P, _P],
    },
    "attention": {
        "zai_paged_attention_general": [_P, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
    },
    "attention_mma": {
        "zai_attention_mma_supports": [_I, _I, _I],
        "zai_prefill_attention_mma": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
        "zai_decode_attention_mma": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
        "zai_decode_attention_fused": [_P, _P, _P, _P, _P, _I, _P, _P, _F, _P, _I, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I,
                                       _F, _I, _I, _I, _I, _P, _P],
        "zai_decode_chunk_keys": [],
        "zai_prefill_block_rows": [],
    },
    "decode_gemm": {
        "zai_skinny_gemm_supports": [_I, _I, _I, _I, _I],
        "zai_skinny_gemm": [_P, _P, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _I, _P],
        "zai_skinny_conv": [_P, _P, _P, _P, _P, _P, _P, _F, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
        "zai_skinny_hint_next": [_P, ctypes.c_longlong],
    },
    "stream_gemm": {
        "zai_stream_gemm_supports": [_I, _I, _I, _I],
        "zai_stream_force_cluster": [_I],
        "zai_stream_force_rows": [_I],
        "zai_stream_debug": [_P],
        "zai_stream_gemm": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
        "zai_stream_conv": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    },
    "gemm_tc": {
        "zai_gemm_tc_supports": [_I, _I, _I, _I],
        "zai_gemm_tc": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
    },
    "gemm_tc_pair": {
        "zai_gemm_pair_supports": [_I, _I, _I, _I],
        "zai_gemm_pair": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    },
    "attention_tma": {
        "zai_decode_attention_tma_supports": [_I, _I, _I, _I],
        "zai_decode_attention_tma": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _F, _P, _I, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I,
                                     _I, _F, _I, _I, _I, _P],
    },
    "attention_tc": {
        "zai_prefill_attention_tc_supports": [_I, _I, _I, _I],
        "zai_prefill_attention_tc": [_P, _P, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P, _P, _P],
        "zai_prefill_attention_tc_splits": [_I, _I, _I, _I],
    },
    "sampling": {
        "zai_argmax": [_P, _P, _I, _I, _P, _P],
        "zai_repetition_penalty": [_P, _P, _P, _P, _P, _I, _I, _P],
        "zai_repetition_penalty_counts": [_P, _P, _P, _P, _P, _I, _I, _P],
        "zai_count_tokens": [_P, _P, _P, _I, _I, _P],
        "zai_sample": [_P, _P, _P, _P, _P, _P, _I, _I, _P, _P],
    },
}

_fns = {}


class KernelError(RuntimeError):
    pass


def _fn(lib_name: str, fn_name: str):
    f = _fns.get(fn_name)
    if f is None:
        lib = build.load(lib_name)
        f = getattr(lib, fn_name)
        f.argtypes = _SIGNATURES[lib_name][fn_name]
        f.restype = c_int
        _fns[fn_name] = f
    return f


launches = 0        # kernels of this package launched so far (a count of launcher calls that ran)


def _check(code: int, what: str, n: int = 1) -> None:
    global launches
    if code == 0:
        launches += n
        return
    if code == -1:
        raise KernelError(f"{what}: element type not supported by the kernel")
    if code == -2:
        raise KernelError(f"{what}: a size is outside what the kernel supports")
    raise KernelError(f"{what}: CUDA error {code} at launch")


CORE_LIBS = ("embed", "norm", "activation", "shortconv", "rope_kv", "attention", "sampling")
BF16_LIBS = ("attention_mma", "attention_tma", "attention_tc", "decode_gemm")


def require(dtype=None) -> None:
    """Fail loudly unless a CUDA device is present and the libraries load that a model of `dtype`
    uses (all of them if no dtype is given).  What is missing or out of date is compiled now, several
    sources at a time; a library outside this set is compiled when it is first called."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this engine has no CPU path")
    libs = list(CORE_LIBS)
    if dtype is None or dtype == torch.bfloat16:
        libs += list(BF16_LIBS)
        if dtype is None or USE_TC_GEMM:
            libs.append("gemm_tc")
        if dtype is None or USE_PAIR_GEMM:
            libs.append("gemm_tc_pair")
        if dtype is None or USE_STREAM_GEMM:
            libs.append("stream_gemm")
    build.build_some(libs, verbose=True)
    for lib in libs:
        build.load(lib)


_SKINNY_VARIANTS = {1: "bf16", 2: "norm, bf16", 3: "f32", 4: "norm, f32", 5: "swiglu", 6: "norm, swiglu", 7: "conv",
                    8: "norm, conv"}


def _kernel_at(lib: str, line: int, cache={}) -> str:
    """The name of the __global__ function whose body holds `line` of csrc/<lib>.cu."""
    import re
    if lib not in cache:
        with open(os.path.join(build.CSRC, lib + ".cu")) as f:
            cache[lib] = f.read().split("\n")
    name = "?"
    for text in cache[lib][:line]:
        m = re.search(r"__global__[^(]*?(\w+)\s*\(", re.sub(r"__(launch_bounds|maxnreg)__\([^)]*\)", "", text))
        if m:
            name = m.group(1)
    return name


def timeline():
    """With libraries built under ZAI_TIMELINE=1: the kernels run since the last call, as a list of
    (kernel, ns when the kernel's first block reached its dependency wait, ns when the wait was
    over) in the order of the second time; marks set inside kernels come as ("<library> mark <n>",
    ns, ns).  Reads the device."""
    import ctypes
    if not build.TIMELINE:
        raise KernelError("the libraries were built without ZAI_TIMELINE=1")
    torch.cuda.synchronize()
    out = []
    buf = (ctypes.c_ulonglong * (3 * 16384))()
    for name in build.sources():
        lib = build.load(name)
        fn = lib.zai_timeline_read
        fn.argtypes = [ctypes.c_void_p, c_int]
        fn.restype = c_int
        n = fn(ctypes.cast(buf, ctypes.c_void_p), 16384)
        if n < 0:
            raise KernelError(f"zai_timeline_read failed in {name}")
        for i in range(n):
            ident, a, b = int(buf[3 * i]), int(buf[3 * i + 1]), int(buf[3 * i + 2])
            if ident >> 32 == 2:
                out.append((f"{name} block {ident & 0xffffffff}", a, b))
            elif ident >> 32:
                out.append((f"{name} mark {ident & 255}", b, b))
            else:
                kernel, variant = _kernel_at(name, ident >> 8), ident & 255
                if name == "decode_gemm" and variant:
                    kernel += f" ({_SKINNY_VARIANTS.get(variant, variant)})"
                out.append((kernel, a, b))
    out.sort(key=lambda r: r[2])
    return out


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"element type {t.dtype} is not supported")


def _ptr(t):
    return None if t is None else t.data_ptr()


_stream_handle = None


def begin_forward() -> None:
    """Called once at the start of a forward pass: the current stream is looked up here and reused by
    every launch of the pass (the lookup costs about as much as a launch)."""
    global _stream_handle
    _stream_handle = torch.cuda.current_stream().cuda_stream


def end_forward() -> None:
    global _stream_handle
    _stream_handle = None


def _stream():
    return _stream_handle if _stream_handle is not None else torch.cuda.current_stream().cuda_stream



def _cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernels take contiguous CUDA tensors")


# ----------------------------------------------------------------------------- timing by kernel class
# The reference prints, per stage of a step, the time its kernels took (PERF_STAGE, src/main.zig:817-931,
# 1369-1412).  Here `profile_begin()` makes every kernel function below record a CUDA event before and
# after its launches under the name of its class; `profile_end()` waits and returns milliseconds per
# class.  No special build is needed; steps must be launched kernel by kernel for it (a replayed graph
# has no place for events), so their sum is larger than a graphed step's time: it is the shares that count.
_profile = None
_profile_depth = 0


def profile_begin() -> None:
    global _profile
    _profile = []


def profile_end() -> dict:
    """Milliseconds per kernel class since `profile_begin()` (waits for the device)."""
    global _profile
    records, _profile = _profile or [], None
    torch.cuda.synchronize()
    out = {}
    for name, a, b in records:
        out[name] = out.get(name, 0.0) + a.elapsed_time(b)
    return out


def _timed(name):
    """Record the decorated kernel function under class `name` while a profile is open (`name` may be a
    function of the call's arguments and result).  A call that launched nothing (returned None) is not
    recorded."""
    def wrap(f):
        import functools

        @functools.wraps(f)
        def g(*args, **kwargs):
            global _profile_depth
            if _profile is None or _profile_depth:             # (a kernel function called by another counts with it)
                return f(*args, **kwargs)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            _profile_depth += 1
            try:
                r = f(*args, **kwargs)
            finally:
                _profile_depth -= 1
            if r is None and f.__name__.startswith("_"):
                return r
            b.record()
            _profile.append((name(*args, **kwargs) if callable(name) else name, a, b))
            return r
        return g
    return wrap


def _product_class(x, w, epilogue, *rest, **kw):
    return {_EPI_F32: "head", _EPI_SWIGLU: "products (gate/up + SwiGLU)", 3: "products (in_proj + conv)"}.get(epilogue, "products")


# ----------------------------------------------------------------------------- kernels
fuses_norm = True       # `linear` and `linear_swiglu` take a LazyNorm and apply it inside the product kernel

_EPI_BF16, _EPI_F32, _EPI_SWIGLU = 0, 1, 2


@_timed("embedding")
def embed(ids, table):
    _cuda(ids, table)
    N, (V, H) = ids.numel(), table.shape
    out = torch.empty((N, H), dtype=torch.float32, device=table.device)
    _check(_fn("embed", "zai_embed")(_ptr(out), _ptr(table), _dt(table), _ptr(ids), N, H, V, _status_ptr(table.device),
                                     _stream()), "embed")
    return out


@_timed("norm")
def gather_add(h, pending, rows):
    _cuda(h, pending, rows)
    R, H = rows.numel(), h.shape[1]
    out = torch.empty((R, H), dtype=torch.float32, device=h.device)
    pd = _dt(pending) if pending is not None else _F32
    _check(_fn("embed", "zai_gather_add")(_ptr(out), _ptr(h), _ptr(pending), pd, _ptr(rows), R, H, _stream()),
           "gather_add")
    return out


@_timed("norm")
def add_rmsnorm(h, delta, w, eps, out_dtype):
    _cuda(h, delta, w)
    if h.dtype != torch.float32 or w.dtype != torch.float32:
        raise KernelError("the residual stream and norm weights are 32-bit")
    N, H = h.shape
    out = torch.empty((N, H), dtype=out_dtype, device=h.device)
    if delta is not None and delta.dtype != out_dtype:
        raise KernelError("the pending term should have the model's dtype")
    _check(_fn("norm", "zai_add_rmsnorm")(_ptr(h), _ptr(delta), _ptr(w), _ptr(out), _dt(out), float(eps), N, H,
                                          _stream()), "add_rmsnorm")
    return out


# ---- which weights follow which.  The few-rows product kernels ask the weights of the product after
# them into L2 while they run.  Nobody has to tell them the order: a call notes that its weights came
# after the last call's, and the next time the last call's weights are used, that is the hint.  (Weak
# references: a hint never outlives the tensor it points to.  A wrong hint, after a change of model
# or of step shape, costs a useless prefetch once and is then replaced.)
_follower = {}          # data_ptr of a weight -> weak reference to the weight used after it last time
_last_weight = [0]


def _hint_next_weights(w) -> None:
    p = w.data_ptr()
    last = _last_weight[0]
    if len(_follower) > 8192:                     # many models have come and gone: start over
        _follower.clear()
    if last and last != p:
        known = _follower.get(last)
        if known is None or known() is not w:
            _follower[last] = weakref.ref(w)
    _last_weight[0] = p
    nxt = _follower.get(p)
    nxt = nxt() if nxt is not None else None
    if nxt is not None and nxt.is_cuda and nxt.device == w.device:
        _fn("decode_gemm", "zai_skinny_hint_next")(nxt.data_ptr(), nxt.numel() * nxt.element_size())


@_timed(_product_class)
def _skinny(x, w, epilogue, out_cols, out_dtype):
    """The few-rows product kernel, if it takes these operands; else None."""
    lazy = isinstance(x, LazyNorm)
    M = (x.rows.numel() if x.rows is not None else x.residual.data.shape[0]) if lazy else x.shape[0]
    O, K = w.shape
    if w.dtype != torch.bfloat16 or (not lazy and x.dtype != torch.bfloat16) or (lazy and x.dtype != torch.bfloat16):
        return None
    if not _fn("decode_gemm", "zai_skinny_gemm_supports")(M, O, K, epilogue, int(lazy)):
        return None
    y = torch.empty((M, out_cols), dtype=out_dtype, device=w.device)
    _hint_next_weights(w)
    if lazy:
        res = x.residual
        _cuda(res.data, x.delta, x.gamma, x.rows)
        h_out = torch.empty_like(res.data) if (x.rows is None and x.delta is not None) else None
        _check(_fn("decode_gemm", "zai_skinny_gemm")(
            _ptr(y), _ptr(w), None, _ptr(res.data), _ptr(x.delta), _ptr(x.gamma), _ptr(x.rows), _ptr(h_out),
            float(x.eps), M, O, K, epilogue, _stream()), "skinny_gemm")
        if h_out is not None:
            res.data = h_out
    else:
        _cuda(x)
        _check(_fn("decode_gemm", "zai_skinny_gemm")(
            _ptr(y), _ptr(w), _ptr(x), None, None, None, None, None, 0.0, M, O, K, epilogue, _stream()), "skinny_gemm")
    return y


TC_MIN_ROWS = 128        # from this many rows on a product may go to the tcgen05 kernel
# Measured on B200 (graph-timed, weights from HBM) the library's two-block 256x256 tiles are 1.15x to
# 2x faster than this one-block 128x{128,256} kernel at the shapes of the LFM2 models, so products go
# to the library unless ZAI_TC_GEMM=1 asks for the tcgen05 kernel (its tests call it directly).
USE_TC_GEMM = os.environ.get("ZAI_TC_GEMM", "0") == "1"

# ---- the status word: one int32 per device that kernels OR bits into (csrc/common.cuh: ZaiStatusBit).
# A kernel that meets an id outside its bound uses id 0 instead, and a kernel whose bounded wait runs
# out stops waiting; both raise a bit here, and whoever reads the step's results reads this word
# with them and throws the step away if it is not zero.
STATUS_BITS = {1: "a bounded wait inside a kernel ran out", 2: "a token id outside the vocabulary",
               4: "a block-table entry outside the page pool", 8: "a state slot outside the slots",
               16: "a position outside its request's block-table row"}
_status = {}


def status_tensor(device=None) -> torch.Tensor:
    """The device's status word (int32 [1]), made at first use."""
    dev = torch.device("cuda") if device is None else torch.device(device)
    index = torch.cuda.current_device() if dev.index is None else dev.index
    entry = _status.get(index)
    if entry is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
        entry = _status[index] = (t, t.data_ptr())
    return entry[0]


def _status_ptr(device) -> int:
    entry = _status.get(device.index)
    if entry is None:
        status_tensor(device)
        entry = _status[torch.cuda.current_device() if device.index is None else device.index]
    return entry[1]


def describe_status(code: int) -> str:
    return "; ".join(text for bit, text in STATUS_BITS.items() if code & bit) or f"status {code}"


def read_status(device=None) -> int:
    """The status word, cleared (reads the device: waits for the work queued so far)."""
    t = status_tensor(device)
    v = int(t.item())
    if v:
        t.zero_()
    return v


def tc_status() -> int:
    """1 if a bounded wait of a kernel ran out since the status word was last read, else 0 (reads the device)."""
    return 1 if read_status() & 1 else 0


@_timed(_product_class)
def _tensor_core(x, w, epilogue, out_cols, out_dtype):
    """The tcgen05 product kernel, if it takes these operands and is the faster choice; else None."""
    N, (O, K) = x.shape[0], w.shape
    if not USE_TC_GEMM or N < TC_MIN_ROWS or w.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
        return None
    if not x.is_contiguous() or not _fn("gemm_tc", "zai_gemm_tc_supports")(N, O, K, epilogue):
        return None
    y = torch.empty((N, out_cols), dtype=out_dtype, device=w.device)
    _check(_fn("gemm_tc", "zai_gemm_tc")(_ptr(y), _ptr(w), _ptr(x), _status_ptr(w.device), N, O, K, epilogue, _stream()),
           "gemm_tc")
    return y


# Steps of 17 to 128 rows: the weight-streaming tcgen05 kernel (csrc/stream_gemm.cu), with SwiGLU or the
# short convolution as its epilogue.  Measured on B200 it is behind the library's product plus the
# separate activation / convolution kernel at the shapes of the LFM2 models (a block's K loop costs about
# 0.4 us per 64-k slice whatever the slice holds: see profiles/stream_gemm_tcgen05_17_128_rows.md), so it
# is an option: ZAI_STREAM_GEMM=1 turns it on.
USE_STREAM_GEMM = os.environ.get("ZAI_STREAM_GEMM", "0") == "1"
STREAM_MIN_ROWS, STREAM_MAX_ROWS = 17, 128


@_timed(_product_class)
def _stream_product(x, w, epilogue, out_cols, out_dtype):
    """The weight-streaming product kernel, if it takes these operands; else None."""
    N, (O, K) = x.shape[0], w.shape
    if (not USE_STREAM_GEMM or not STREAM_MIN_ROWS <= N <= STREAM_MAX_ROWS or w.dtype != torch.bfloat16
            or x.dtype != torch.bfloat16 or not x.is_contiguous() or not w.is_contiguous()):
        return None
    if not _fn("stream_gemm", "zai_stream_gemm_supports")(N, O, K, epilogue):
        return None
    y = torch.empty((N, out_cols), dtype=out_dtype, device=w.device)
    _check(_fn("stream_gemm", "zai_stream_gemm")(_ptr(y), _ptr(w), _ptr(x), _status_ptr(w.device), N, O, K, epilogue,
                                                 _stream()), "stream_gemm")
    return y


def linear(x, w, out_dtype=None):
    """x [N, K] times w [O, K] transposed.  x may be a LazyNorm.  Few rows in bfloat16 go to the
    fused few-rows kernel, many rows to the tcgen05 kernel where it is the faster one; a matrix kept
    in 32-bit is multiplied in 32-bit; the rest is the library's."""
    in_dtype = x.dtype
    out_dtype = out_dtype or in_dtype
    if in_dtype == torch.bfloat16 and out_dtype in (torch.bfloat16, torch.float32):
        y = _skinny(x, w, _EPI_F32 if out_dtype == torch.float32 else _EPI_BF16, w.shape[0], out_dtype)
        if y is not None:
            return y
    if isinstance(x, LazyNorm):
        x = x.materialize(sys.modules[__name__])
    if x.dtype == torch.bfloat16 and out_dtype in (torch.bfloat16, torch.float32):
        epi = _EPI_F32 if out_dtype == torch.float32 else _EPI_BF16
        y = _stream_product(x, w, epi, w.shape[0], out_dtype)
        if y is None:
            y = _tensor_core(x, w, epi, w.shape[0], out_dtype)
        if y is not None:
            return y
    return _library_product(x, w, out_dtype)


@_timed(lambda x, w, out_dtype: "head" if out_dtype == torch.float32 and x.dtype != torch.float32 else "products")
def _library_product(x, w, out_dtype):
    """The library's matrix product: true 32-bit where an operand or the result is 32-bit."""
    if x.dtype == torch.float32 or w.dtype == torch.float32 or out_dtype == torch.float32:
        if torch.backends.cuda.matmul.allow_tf32:
            torch.backends.cuda.matmul.allow_tf32 = False
        if x.dtype == w.dtype == torch.bfloat16:
            # 32-bit logits from 16-bit operands: the product itself accumulates in 32-bit
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.matmul(x.float(), w.float().t()).to(out_dtype)
    return torch.matmul(x, w.t())


# The two-block tcgen05 kernel (csrc/gemm_tc_pair.cu) runs the gate/up product with SwiGLU in its
# epilogue in the time the library's product and the activation kernel take together where the model is
# 1024 wide (a prefill of 2048 tokens at the 350M shape: 1.98-2.01 ms either way, measured in one run)
# and is 1 % and 2 % behind them at the widths of the 700M and 1.2B shapes.  So gate/up products of
# PAIR_SWIGLU_MIN_ROWS rows or more go to it where K is at most PAIR_SWIGLU_MAX_K; ZAI_PAIR_GEMM=1 sends
# them there at every width, ZAI_PAIR_GEMM=0 never.
PAIR_SWIGLU_MIN_ROWS = int(os.environ.get("ZAI_PAIR_SWIGLU_MIN_ROWS", "1024"))
PAIR_SWIGLU_MAX_K = 1024
_pair_env = os.environ.get("ZAI_PAIR_GEMM", "auto")
USE_PAIR_GEMM = _pair_env != "0"             # False: never; True: by the rule above (or always, with PAIR_GEMM_ALWAYS)
PAIR_GEMM_ALWAYS = _pair_env == "1"


@_timed(_product_class)
def gemm_pair(x, w, epilogue, out_cols, out_dtype, wide=-1):
    """The two-block tcgen05 product kernel: x [N, K] times w [O, K] transposed with the epilogue
    (0 bfloat16, 1 32-bit, 2 SwiGLU over stacked gate|up rows); None if it does not take the operands."""
    _cuda(x, w)
    N, (O, K) = x.shape[0], w.shape
    if w.dtype != torch.bfloat16 or x.dtype != torch.bfloat16 or not x.is_contiguous() or not w.is_contiguous():
        return None
    if not _fn("gemm_tc_pair", "zai_gemm_pair_supports")(N, O, K, epilogue):
        return None
    y = torch.empty((N, out_cols), dtype=out_dtype, device=w.device)
    _check(_fn("gemm_tc_pair", "zai_gemm_pair")(_ptr(y), _ptr(w), _ptr(x), _status_ptr(w.device), N, O, K, epilogue, wide,
                                                _stream()), "gemm_pair")
    return y


def linear_swiglu(x, w_gate_up, ff_dim):
    """silu(x . Wgate^T) * (x . Wup^T) with the two matrices stacked as [2F, K]."""
    if x.dtype == torch.bfloat16:
        y = _skinny(x, w_gate_up, _EPI_SWIGLU, ff_dim, torch.bfloat16)
        if y is not None:
            return y
        if isinstance(x, LazyNorm):
            x = x.materialize(sys.modules[__name__])
        y = _stream_product(x, w_gate_up, _EPI_SWIGLU, ff_dim, torch.bfloat16)
        if y is None:
            y = _tensor_core(x, w_gate_up, _EPI_SWIGLU, ff_dim, torch.bfloat16)
        if y is not None:
            return y
        if USE_PAIR_GEMM and x.shape[0] >= PAIR_SWIGLU_MIN_ROWS and (PAIR_GEMM_ALWAYS or x.shape[1] <= PAIR_SWIGLU_MAX_K):
            y = gemm_pair(x, w_gate_up, _EPI_SWIGLU, ff_dim, torch.bfloat16)
            if y is not None:
                return y
    return silu_mul(linear(x, w_gate_up), ff_dim)


@_timed("activation")
def silu_mul(gu, ff_dim):
    _cuda(gu)
    N = gu.shape[0]
    out = torch.empty((N, ff_dim), dtype=gu.dtype, device=gu.device)
    _check(_fn("activation", "zai_silu_mul")(_ptr(out), _ptr(gu), _dt(gu), N, ff_dim, _stream()), "silu_mul")
    return out


_EPI_CONV = 3
FUSED_CONV_MAX_TAPS = 4


def linear_short_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state=True):
    """z = C * conv(state ++ B * x~) with (B, C, x~) = x . w_in^T: the short convolution's input
    projection, gates, taps and state update.  A step of single tokens (at most 16) runs as one
    kernel, the convolution being the product's epilogue; other steps as the product and the
    convolution kernel."""
    lazy = isinstance(x, LazyNorm)
    M = (x.rows.numel() if x.rows is not None else x.residual.data.shape[0]) if lazy else x.shape[0]
    O, K = w_in.shape
    C = O // 3
    fused = (step.decode_only and taps <= FUSED_CONV_MAX_TAPS and w_in.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
             and (not lazy or x.rows is None) and state.dtype == torch.float32 and state.shape[-1] == C
             and M == step.n_seqs and _fn("decode_gemm", "zai_skinny_gemm_supports")(M, O, K, _EPI_CONV, int(lazy)))
    if not fused:
        if (USE_STREAM_GEMM and step.decode_only and STREAM_MIN_ROWS <= M <= STREAM_MAX_ROWS and M == step.n_seqs
                and taps <= FUSED_CONV_MAX_TAPS and w_in.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
                and (not lazy or x.rows is None) and state.dtype == torch.float32 and state.shape[-1] == C and w_in.is_contiguous()
                and _fn("stream_gemm", "zai_stream_gemm_supports")(M, O, K, _EPI_CONV)):
            if lazy:
                x = x.materialize(sys.modules[__name__])
            return _stream_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state, M, C, K)
        return short_conv(linear(x, w_in), conv_w, conv_b, state, step, taps, write_state)
    return _skinny_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state, lazy, M, C, K)


@_timed("products (in_proj + conv)")
def _stream_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state, M, C, K):
    _cuda(x, w_in, conv_w, conv_b, state)
    z = torch.empty((M, C), dtype=torch.bfloat16, device=w_in.device)
    _check(_fn("stream_gemm", "zai_stream_conv")(
        _ptr(z), _ptr(w_in), _ptr(x), _status_ptr(w_in.device), _ptr(conv_w), _ptr(conv_b), _ptr(state), _ptr(step.slot_ids),
        M, C, K, int(taps), state.shape[1], int(bool(write_state)), state.shape[0], _stream()), "stream_conv")
    return z


@_timed("products (in_proj + conv)")
def _skinny_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state, lazy, M, C, K):
    _cuda(w_in, conv_w, conv_b, state)
    z = torch.empty((M, C), dtype=torch.bfloat16, device=w_in.device)
    fn = _fn("decode_gemm", "zai_skinny_conv")
    _hint_next_weights(w_in)
    tail = (_ptr(conv_w), _ptr(conv_b), _ptr(state), _ptr(step.slot_ids), M, C, K, int(taps), state.shape[1],
            int(bool(write_state)), state.shape[0], _status_ptr(state.device), _stream())
    if lazy:
        res = x.residual
        _cuda(res.data, x.delta, x.gamma)
        h_out = torch.empty_like(res.data) if x.delta is not None else None
        _check(fn(_ptr(z), _ptr(w_in), None, _ptr(res.data), _ptr(x.delta), _ptr(x.gamma), _ptr(h_out), float(x.eps), *tail),
               "skinny_conv")
        if h_out is not None:
            res.data = h_out
    else:
        _cuda(x)
        _check(fn(_ptr(z), _ptr(w_in), _ptr(x), None, None, None, None, 0.0, *tail), "skinny_conv")
    return z


@_timed("conv")
def short_conv(bcx, conv_w, conv_b, state, step, taps, write_state=True):
    _cuda(bcx, conv_w, conv_b, state)
    N, C = bcx.shape[0], bcx.shape[1] // 3
    z = torch.empty((N, C), dtype=bcx.dtype, device=bcx.device)
    if state.dtype != torch.float32 or state.shape[-1] != C:
        raise KernelError("the conv state is 32-bit [slots, rows, channels]")
    _check(_fn("shortconv", "zai_short_conv")(
        _ptr(z), _ptr(bcx), _dt(bcx), _ptr(conv_w), _ptr(conv_b), _ptr(state), _ptr(step.seq_idx), _ptr(step.cu_q),
        _ptr(step.slot_ids), N, step.n_seqs, C, int(taps), state.shape[1], int(step.decode_only),
        int(write_state), state.shape[0], _status_ptr(state.device), _stream()), "short_conv", 1 if (step.decode_only or taps == 1 or not write_state) else 2)
    return z


_inv_freq_cache = {}


def inverse_frequencies(rotary_dim: int, theta: float, device) -> torch.Tensor:
    """theta^(-2i/n) for i < n/2, computed in 64-bit."""
    key = (rotary_dim, float(theta), str(device))
    t = _inv_freq_cache.get(key)
    if t is None:
        i = torch.arange(rotary_dim // 2, dtype=torch.float64)
        t = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / rotary_dim).to(device)
        _inv_freq_cache[key] = t
    return t


@_timed("q/k norm, rotation, page write")
def rope_table(step, rotary_dim: int, theta: float, device) -> torch.Tensor:
    """(cos, sin) of position * frequency for every row of the step, [N, rotary_dim/2, 2] 32-bit,
    computed once per step and rotation and kept with the step."""
    key = ("rope", rotary_dim, float(theta))
    t = step.scratch.get(key)
    if t is None:
        half = rotary_dim // 2
        t = torch.empty((step.n_tokens, half, 2), dtype=torch.float32, device=device)
        _check(_fn("rope_kv", "zai_rope_table")(_ptr(t), _ptr(step.positions), _ptr(inverse_frequencies(rotary_dim, theta, device)),
                                                step.n_tokens, half, _stream()), "rope_table")
        step.scratch[key] = t
    return t


@_timed("q/k norm, rotation, page write")
def qk_norm_rope(qkv, q_w, k_w, eps, rotary_dim, theta, step, cache, heads, kv_heads, head_dim,
                 has_kv=True, write=True, return_k=False):
    _cuda(qkv, q_w, k_w)
    N, cols = qkv.shape
    q = torch.empty((N, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    k_out = torch.empty((N, kv_heads * head_dim), dtype=qkv.dtype, device=qkv.device) if (return_k and has_kv) else None
    table = rope_table(step, rotary_dim, theta, qkv.device) if rotary_dim else None
    do_write = bool(write and has_kv)
    pages, bt = cache.pages, cache.block_table
    if do_write and pages.dtype != qkv.dtype:
        raise KernelError("the pages and the activations should have one dtype")
    _check(_fn("rope_kv", "zai_qk_norm_rope")(
        _ptr(qkv), cols, _dt(qkv), _ptr(q_w), _ptr(k_w), float(eps), _ptr(table), int(rotary_dim),
        _ptr(step.positions), _ptr(step.seq_idx), _ptr(bt) if do_write else None,
        bt.shape[1] if do_write else 0, _ptr(pages) if do_write else None, cache.page_size, _ptr(q), _ptr(k_out),
        N, heads, kv_heads, head_dim, int(has_kv), int(do_write), pages.shape[0] if do_write else 0,
        _status_ptr(qkv.device), _stream()), "qk_norm_rope")
    return q, k_out


@_timed("q/k norm, rotation, page write")
def kv_write(k, v, step, cache, kv_heads, head_dim):
    if k.stride(-1) != 1 or v.stride(-1) != 1:
        raise KernelError("k and v rows should be contiguous")
    N = k.shape[0]
    _check(_fn("rope_kv", "zai_kv_write")(
        _ptr(k), k.stride(0), _ptr(v), v.stride(0), _dt(k), _ptr(step.positions), _ptr(step.seq_idx),
        _ptr(cache.block_table), cache.block_table.shape[1], _ptr(cache.pages), cache.page_size, N, kv_heads,
        head_dim, cache.pages.shape[0], _status_ptr(k.device), _stream()), "kv_write")


USE_TC_ATTENTION = os.environ.get("ZAI_TC_ATTENTION", "1") == "1"     # tcgen05 prefill attention where the sizes allow



_span_tickets = {}


def _attention_tickets(device, n):
    """Zeroed counters for the span attention's shared tiles (the kernel leaves them zero)."""
    t = _span_tickets.get(device)
    if t is None or t.numel() < n:
        t = torch.zeros((max(n, 1024),), dtype=torch.int32, device=device)
        _span_tickets[device] = t
    return t

@_timed("attention")
def paged_attention(q, step, cache, heads, kv_heads, head_dim, scale, window=None, impl=None):
    """Causal attention of the step's rows over their requests' pages.  bfloat16 runs on the
    tensor cores (a split-key kernel when every span is one token, else the flash-style kernel)
    for the head sizes those kernels have; everything else, and `impl="general"`, runs the
    general kernel.  `impl="mma"` / `impl="tcgen05"` pick between the two span kernels."""
    _cuda(q)
    N = q.shape[0]
    if N != step.n_tokens:
        raise KernelError(f"{N} query rows for a step of {step.n_tokens} rows")
    out = torch.empty((N, heads * head_dim), dtype=q.dtype, device=q.device)
    if cache.pages.dtype != q.dtype:
        raise KernelError("the pages and the queries should have one dtype")
    bt = cache.block_table
    if (impl != "general" and q.dtype == torch.bfloat16
            and _fn("attention_mma", "zai_attention_mma_supports")(head_dim, heads, kv_heads)):
        def single_tokens(n):
            # rows 0..n-1 are one token each, row i of span i: keys split over blocks, then combined
            chunk = _fn("attention_mma", "zai_decode_chunk_keys")()
            n_chunks = max(-(-int(step.max_kv_len) // chunk), 1)
            part_o = torch.empty((n, heads, n_chunks, head_dim), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((n, heads, n_chunks, 2), dtype=torch.float32, device=q.device)
            _check(_fn("attention_mma", "zai_decode_attention_mma")(
                _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(q), _ptr(cache.pages), _ptr(bt), bt.shape[1],
                _ptr(step.positions), n, n_chunks, cache.page_size, heads, kv_heads, head_dim, float(scale),
                int(window or 0), cache.pages.shape[0], _status_ptr(q.device), _stream()), "decode attention", 2)

        if step.decode_only:
            single_tokens(N)
        else:
            # the one-token spans at the front of a mixed step (decoding requests beside prompt portions)
            # would each fill a whole block of query rows of the span kernel: they go to the other one
            ns = int(getattr(step, "single_first", 0)) if (SPLIT_MIXED_ATTENTION and q.is_contiguous()) else 0
            if ns:
                single_tokens(ns)
            S = step.n_seqs - ns
            cu_q, ctx_lens, bt = step.cu_q[ns:], step.ctx_lens[ns:], bt[ns:]
            block_rows = _fn("attention_mma", "zai_prefill_block_rows")()
            n_tiles = (step.attn_tiles - ns) if getattr(step, "attn_tiles", None) else sum(-(-n // block_rows) for n in step.q_lens[ns:])
            if (impl != "mma" and (USE_TC_ATTENTION or impl == "tcgen05") and q.is_contiguous()
                    and _fn("attention_tc", "zai_prefill_attention_tc_supports")(head_dim, heads, kv_heads, cache.page_size)):
                # few tiles of query rows over long contexts: several blocks share a tile's keys and leave their
                # parts in scratch, the last to finish combines them (tickets: zero before and after)
                splits = _fn("attention_tc", "zai_prefill_attention_tc_splits")(n_tiles, heads, bt.shape[1], cache.page_size)
                part_o = part_ml = None
                tickets = _attention_tickets(q.device, n_tiles * heads if splits > 1 else 0)   # (made at the first call, which no graph captures)
                if splits > 1:
                    part_o = torch.empty((n_tiles * heads * splits, 64 * 128), dtype=torch.float32, device=q.device)
                    part_ml = torch.empty((n_tiles * heads * splits, 2 * 128), dtype=torch.float32, device=q.device)
                _check(_fn("attention_tc", "zai_prefill_attention_tc")(
                    _ptr(out), _ptr(q), _ptr(cache.pages), cache.pages.shape[0], _status_ptr(q.device), _ptr(bt), bt.shape[1],
                    _ptr(cu_q), _ptr(ctx_lens), N, S, n_tiles, cache.page_size, heads, kv_heads,
                    head_dim, float(scale), int(window or 0), splits, _ptr(part_o), _ptr(part_ml), _ptr(tickets),
                    _stream()), "prefill attention (tcgen05)")
                return out
            _check(_fn("attention_mma", "zai_prefill_attention_mma")(
                _ptr(out), _ptr(q), _ptr(cache.pages), _ptr(bt), bt.shape[1], _ptr(cu_q), _ptr(ctx_lens),
                S, n_tiles, cache.page_size, heads, kv_heads, head_dim, float(scale), int(window or 0),
                cache.pages.shape[0], _status_ptr(q.device), _stream()), "prefill attention")
        return out
    _check(_fn("attention", "zai_paged_attention_general")(
        _ptr(out), _ptr(q), _ptr(cache.pages), _dt(q), _ptr(bt), bt.shape[1],
        _ptr(step.positions), _ptr(step.seq_idx), cache.page_size, N, heads, kv_heads, head_dim, float(scale),
        int(window or 0), cache.pages.shape[0], _status_ptr(q.device), _stream()), "paged_attention")
    return out


_tickets = {}
SPLIT_MIXED_ATTENTION = os.environ.get("ZAI_SPLIT_MIXED_ATTENTION", "1") == "1"
USE_TMA_ATTENTION = os.environ.get("ZAI_TMA_ATTENTION", "1") == "1"   # keys and values by TMA where the sizes allow
DECODE_BLOCKS_WANTED = 500


def fused_decode_attention_available(dtype, heads, kv_heads, head_dim) -> bool:
    return dtype == torch.bfloat16 and bool(_fn("attention_mma", "zai_attention_mma_supports")(head_dim, heads, kv_heads))


@_timed("attention (with q/k norm, rotation, page write)")
def decode_attention_fused(qkv, q_w, k_w, eps, rotary_dim, theta, step, cache, heads, kv_heads, head_dim, scale,
                           window=None, write=True):
    """A decode step's attention in one kernel, from the qkv projection's rows [B, (Hq + 2 Hkv) D]:
    q/k RMSNorm, rotation, the new key and value into their page, attention over the pages in chunks
    of keys, and the combination of the chunks.  Every row of the step is one token."""
    _cuda(qkv, q_w, k_w)
    B, cols = qkv.shape
    if B != step.n_tokens:
        raise KernelError(f"{B} rows for a step of {step.n_tokens} rows")
    dev = qkv.device
    out = torch.empty((B, heads * head_dim), dtype=qkv.dtype, device=dev)
    # keys per block: about DECODE_BLOCKS_WANTED blocks (a little more than the SMs hold at once), so
    # that a block's start-up and its partial sums are spread over many keys without leaving SMs
    # idle (a power of two between 256 and 1024)
    want = int(step.max_kv_len) * B * kv_heads // DECODE_BLOCKS_WANTED
    chunk = 256
    while chunk < 1024 and chunk * 3 < want * 2:
        chunk *= 2
    chunk = int(os.environ.get("ZAI_DECODE_CHUNK", chunk))
    n_chunks = max(-(-int(step.max_kv_len) // chunk), 1)
    part_o = torch.empty((B, heads, n_chunks, head_dim), dtype=torch.float32, device=dev)
    part_ml = torch.empty((B, heads, n_chunks, 2), dtype=torch.float32, device=dev)
    tickets = _tickets.get(str(dev))
    if tickets is None or tickets.numel() < B * kv_heads:
        tickets = torch.zeros(max(B * kv_heads, 65536), dtype=torch.int32, device=dev)
        _tickets[str(dev)] = tickets
    table = rope_table(step, rotary_dim, theta, dev) if rotary_dim else None
    bt = cache.block_table
    if USE_TMA_ATTENTION and _fn("attention_tma", "zai_decode_attention_tma_supports")(head_dim, heads, kv_heads, cache.page_size):
        _check(_fn("attention_tma", "zai_decode_attention_tma")(
            _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(tickets), _status_ptr(dev), _ptr(qkv), cols, _ptr(q_w), _ptr(k_w),
            float(eps), _ptr(table), int(rotary_dim), _ptr(cache.pages), cache.pages.shape[0], _ptr(bt), bt.shape[1],
            _ptr(step.positions), B, n_chunks, cache.page_size, heads, kv_heads, head_dim, float(scale), int(window or 0),
            int(bool(write)), chunk, _stream()), "decode_attention_tma")
        return out
    _check(_fn("attention_mma", "zai_decode_attention_fused")(
        _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(tickets), _ptr(qkv), cols, _ptr(q_w), _ptr(k_w), float(eps),
        _ptr(table), int(rotary_dim), _ptr(cache.pages), _ptr(bt), bt.shape[1], _ptr(step.positions), B, n_chunks,
        cache.page_size, heads, kv_heads, head_dim, float(scale), int(window or 0), int(bool(write)), chunk,
        cache.pages.shape[0], _status_ptr(dev), _stream()), "decode_attention_fused")
    return out


@_timed("sampling")
def argmax(logits, with_status=False):
    """First index of each row's maximum, int32 [R]; `with_status`: [R + 1], the device's status word behind
    the ids (one copy to the host then brings both)."""
    _cuda(logits)
    R, V = logits.shape
    out = torch.empty((R + (1 if with_status else 0),), dtype=torch.int32, device=logits.device)
    _check(_fn("sampling", "zai_argmax")(_ptr(out), _ptr(logits), R, V,
                                         _status_ptr(logits.device) if with_status else None, _stream()), "argmax")
    return out


@_timed("sampling")
def repetition_penalty(logits, tokens, counts, offsets, penalty):
    """In place: logits[r, tokens[i]] is penalised counts[i] times for offsets[r] <= i < offsets[r+1]."""
    _cuda(logits, tokens, counts, offsets, penalty)
    R, V = logits.shape
    _check(_fn("sampling", "zai_repetition_penalty")(_ptr(logits), _ptr(tokens), _ptr(counts), _ptr(offsets),
                                                     _ptr(penalty), R, V, _stream()), "repetition_penalty")
    return logits


@_timed("sampling")
def repetition_penalty_counts(logits, counts, slots, penalty):
    """A copy of logits [R, V] with the repetition penalty applied from a table of counts [slots, V] on the
    device (slots [R] int32, negative: the row has none)."""
    _cuda(logits, counts, slots, penalty)
    R, V = logits.shape
    if counts.dtype != torch.int32 or counts.shape[1] != V or logits.dtype != torch.float32:
        raise KernelError("the penalty takes 32-bit logits and int32 counts [slots, vocabulary]")
    out = torch.empty_like(logits)
    _check(_fn("sampling", "zai_repetition_penalty_counts")(_ptr(out), _ptr(logits), _ptr(counts), _ptr(slots), _ptr(penalty),
                                                           R, V, _stream()), "repetition_penalty_counts")
    return out


@_timed("sampling")
def count_tokens(counts, ids, slots, rows):
    """counts[slots[r], ids[r]] += 1 for the first `rows` rows that have a slot."""
    _cuda(counts, ids, slots)
    _check(_fn("sampling", "zai_count_tokens")(_ptr(counts), _ptr(ids), _ptr(slots), int(rows), counts.shape[1], _stream()),
           "count_tokens")


@_timed("sampling")
def sample(logits, temperature, top_k, top_p, u, with_status=False):
    _cuda(logits, temperature, top_k, top_p, u)
    R, V = logits.shape
    out = torch.empty((R + (1 if with_status else 0),), dtype=torch.int32, device=logits.device)
    _check(_fn("sampling", "zai_sample")(_ptr(out), _ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                         _ptr(u), R, V, _status_ptr(logits.device) if with_status else None, _stream()), "sample")
    return out
