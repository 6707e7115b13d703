"""The decode-attention entry point that allocates nothing (csrc/attention_no_alloc.h), called
through its exported C symbol as a program without PyTorch's allocator would call it, and compared
with the regular entry point on two calls in a row.

Such a caller owns every buffer it passes and has nowhere to get scratch from at call time (no
caching allocator, a device already handed to its own arena, or a loop in which cudaMalloc's
device-wide synchronisation is not acceptable); the library's static array stands in.  The file is
named to be collected last, so that a run that stops at the first failure has run everything else.
"""
import ctypes
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

ARGS = [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_void_p] + [ctypes.c_int] * 6 + [ctypes.c_float, ctypes.c_int,
                                                                                        ctypes.c_void_p]


def symbol():
    from zig_ai_b200.kernels import build
    lib = build.load("attention_mma")
    fn = lib.zai_decode_attention_static
    fn.argtypes, fn.restype = ARGS, ctypes.c_int
    msg = lib.zai_decode_attention_static_error
    msg.argtypes, msg.restype = [ctypes.c_int], ctypes.c_char_p
    return fn, msg


def make_case(B, Hq, Hkv, D, ps, contexts, seed):
    from test_gpu_kernels import fill_pages, make_step
    from zig_ai_b200.cache.manager import CacheView
    from zig_ai_b200.kernels import ops
    ops.require()
    g = torch.Generator().manual_seed(seed)
    step = make_step(ops, torch.bfloat16, contexts, [1] * B, ps, 1024, seed)
    pages = fill_pages(step, contexts, [1] * B, ps, Hkv, D, torch.bfloat16, 1024, g)
    q = torch.randn(B, Hq * D, generator=g).to(torch.bfloat16).cuda()
    return ops, step, CacheView(0, pages, step.block_tables[0], ps), q


def call_static(fn, q, step, view, Hq, Hkv, D, n_chunks, window=0):
    out = torch.full((q.shape[0], Hq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
    bt = view.block_table
    code = fn(out.data_ptr(), q.data_ptr(), view.pages.data_ptr(), bt.data_ptr(), bt.shape[1],
              step.positions.data_ptr(), q.shape[0], n_chunks, view.page_size, Hq, Hkv, D, D ** -0.5, window,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return code, out


def test_static_scratch_entry_point_matches_the_regular_one_twice():
    fn, msg = symbol()
    # first call: long contexts, many chunks; second call: other sizes, fewer chunks, so that
    # whatever the first call left in the array lies where the second must not read it
    for B, Hq, Hkv, D, ps, contexts, seed in [
        (6, 16, 8, 64, 16, [0, 255, 256, 1030, 2047, 700], 41),
        (3, 6, 2, 96, 8, [5, 300, 63], 42),
    ]:
        ops, step, view, q = make_case(B, Hq, Hkv, D, ps, contexts, seed)
        n_chunks = -(-step.max_kv_len // 256)
        want = ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None)
        code, got = call_static(fn, q, step, view, Hq, Hkv, D, n_chunks)
        assert code == 0, msg(code)
        assert not torch.isnan(got.float()).any()
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        # and against the plain PyTorch version, like the regular kernel in its own test
        import ref_ops
        ref = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None)
        assert torch.allclose(got.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    fn, msg = symbol()
    ops, step, view, q = make_case(2, 16, 8, 64, 16, [10, 20], 43)
    code, out = call_static(fn, q, step, view, 16, 8, 64, n_chunks=(1 << 20) // (2 * 16 * 66) + 1)
    assert code == -3 and b"scratch" in msg(code)
    assert torch.isnan(out.float()).all()                 # nothing was launched
    code, _ = call_static(fn, q, step, view, 16, 8, 64, n_chunks=1)
    assert code == 0
    # a head count of zero is a size the kernel does not take: refused before any arithmetic with it
    code, out = call_static(fn, q, step, view, 16, 0, 64, n_chunks=1)
    assert code == -2 and b"size" in msg(code)
    assert torch.isnan(out.float()).all()
