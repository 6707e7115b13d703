"""The step function: run a batch of (request, its next tokens) from the cache and return the
logits at the wanted places.

The reference's driver loops the layers for one sequence, a prompt chunk or one token at a time
(src/main.zig:832-865 and :1138-1217).  Here one call runs, as one flattened batch, prompt
portions of some requests beside single decoded tokens of others; it runs only the tokens it is
given, reads everything earlier from the cache, and computes the head only where logits are
wanted.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import os

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages
from ..cache.manager import NULL_PAGE, NULL_SLOT
from ..models import build_model
from .batch import StepBatch, pack_step


class StepError(ValueError):
    """A step that cannot run (an unknown token id, a request that is too long, a bad entry), or a step
    whose kernels raised the status word: its results are void."""


class ModelRunner:
    """Owns the model's tensors and the cache, and runs steps."""

    def __init__(self, model, cache: CacheManager, ops, dtype: torch.dtype, device):
        self.model, self.cache, self.ops, self.dtype, self.device = model, cache, ops, dtype, device
        self.processed: Dict[object, int] = {}      # request -> tokens in the cache
        self.steps = 0
        self.tokens_run = 0
        self.graphs = None
        self.shape_graphs = None
        self.use_graphs = False

    def enable_graphs(self, max_positions: int) -> bool:
        """Run decode-only steps as CUDA graphs, if the device is CUDA and every part says its
        forward can be captured (no host reads of device data)."""
        if self.device.type != "cuda" or not all(getattr(p, "graph_safe", False) for p in self.model.all_parts()):
            return False
        from .graph import DecodeGraphs, ShapeGraphs
        self.graphs = DecodeGraphs(self.model, self.cache, self.ops, self.dtype, self.device,
                                   min(max_positions, self.cache.num_pages * self.cache.page_size))
        self.shape_graphs = ShapeGraphs(self.model, self.cache, self.ops, self.dtype, self.device, self.graphs.widths)
        self.use_graphs = True
        return True

    # ------------------------------------------------------------------ requests
    def add_request(self, request_id) -> None:
        self.cache.admit(request_id)
        self.processed[request_id] = 0

    admit = add_request

    def release(self, request_id) -> None:
        self.end_request(request_id)

    def has_request(self, request_id) -> bool:
        return request_id in self.processed

    def end_request(self, request_id) -> None:
        self.cache.release(request_id)
        del self.processed[request_id]

    # ------------------------------------------------------------------ the step
    def _reserve(self, entries: Sequence[Tuple[object, Sequence[int], Sequence[int]]], trusted: bool = False):
        """Check the entries and reserve their pages (all or none).  Returns the spans
        (request, ctx_len, tokens, wanted, slot) and the requests' block tables by group.
        `trusted`: the caller (the scheduler) has checked the tokens and reserved the pages."""
        if not entries:
            raise StepError("a step needs at least one entry")
        if not trusted:
            seen = set()
            V, max_pos = self.model.vocab_size, self.model.spec.max_positions
            for rid, tokens, _want in entries:
                if rid in seen:
                    raise StepError(f"request {rid!r} appears twice in one step")
                seen.add(rid)
                if rid not in self.processed:
                    raise StepError(f"request {rid!r} was not added")
                if len(tokens) < 1:
                    raise StepError(f"request {rid!r} brings no tokens")
                arr = np.asarray(tokens)
                if arr.dtype.kind not in "iu" or arr.min() < 0 or arr.max() >= V:
                    bad = [int(t) for t in tokens if not 0 <= int(t) < V]
                    raise StepError(f"request {rid!r}: token ids {bad[:8]} are outside the vocabulary of {V}")
                if self.processed[rid] + len(tokens) > max_pos:
                    raise StepError(f"request {rid!r} would reach {self.processed[rid] + len(tokens)} positions; "
                                    f"the model allows {max_pos}")
            # all-or-nothing reservation over the whole step
            demand: Dict[int, int] = {}
            for rid, tokens, _want in entries:
                if self.cache._fits_already(self.cache.requests[rid], self.processed[rid] + len(tokens)):
                    continue
                for g, n in self.cache.pages_to_take(rid, self.processed[rid] + len(tokens)).items():
                    demand[g] = demand.get(g, 0) + n
            for g, n in demand.items():
                if n > self.cache.groups[g].pool.n_free:
                    raise OutOfPages(f"the step needs {n} more pages of group {g}; "
                                     f"{self.cache.groups[g].pool.n_free} are free")
            for rid, tokens, _want in entries:
                self.cache.reserve(rid, self.processed[rid] + len(tokens))
        requests = self.cache.requests
        spans = [(rid, self.processed[rid], tokens, want, requests[rid].slot) for rid, tokens, want in entries]
        rids = [e[0] for e in entries]
        ps = self.cache.page_size
        longest = max(self.processed[rid] + len(tokens) for rid, tokens, _ in entries)
        width = max(-(-longest // ps), 1)
        tables = {g: self.cache.table_rows(rids, g, width) for g in self.cache.paged_groups()}
        return spans, tables

    def prepare(self, entries) -> StepBatch:
        spans, tables = self._reserve(entries)
        return pack_step(self.ops, self.dtype, self.device, spans, tables, pin=True)

    def prepare_decode(self, entries):
        """Reserve and pack a single-token step now, to run it later with `run_prepared` (lets a
        caller take the host work out of a timed region).  The requests advance at once."""
        if not self.use_graphs:
            raise StepError("prepared steps need the graph path")
        spans, tables = self._reserve(entries)
        for rid, tokens, _ in entries:
            self.processed[rid] += len(tokens)
        return self.graphs.prepare(spans, tables)

    def run_prepared(self, prepared) -> torch.Tensor:
        self.steps += 1
        self.tokens_run += prepared[1]
        return self.graphs.run_prepared(prepared)

    def _pad_rows(self, spans, tables):
        """Round a step's row count up (see `pad_rows`) on the device path."""
        if self.device.type != "cuda" or os.environ.get("ZAI_PAD_ROWS", "1") == "0":
            return spans, tables
        return pad_rows(spans, tables, self.cache.page_size)

    def can_take_device_tokens(self, n_rows: int) -> bool:
        """Whether a step of `n_rows` single tokens may get its tokens from a device tensor."""
        return bool(self.use_graphs and self.graphs.bucket(n_rows) is not None)

    def check_status(self, step_number: Optional[int] = None) -> None:
        """Read the kernels' status word (this waits for the device) and raise `StepError` if a kernel
        met an id outside its bound or gave up a bounded wait: what the step returned is void.  The
        reference lets every failure of a step come up as an error in the same way
        (src/paged_attention/block_table.zig:37, src/main.zig:394-402)."""
        read = getattr(self.ops, "read_status", None)
        code = read(self.device) if read else 0
        if code:
            raise StepError(f"step {self.steps if step_number is None else step_number}: "
                            f"{self.ops.describe_status(code)} (status {code}); its results are void")

    def step(self, entries, trusted: bool = False, device_tokens: Optional[torch.Tensor] = None,
             check: bool = True) -> torch.Tensor:
        """entries: (request, its next tokens, wanted places among them).  Returns 32-bit logits
        [wanted, vocab] in the order of the entries and of their wanted places.  (A step that ran
        as a CUDA graph returns a view of that graph's output buffer, valid until the next such step.)
        `device_tokens`: for a step of single tokens, the tokens as an int32 device tensor in the
        order of the entries; the tokens in `entries` are then placeholders.
        `check`: read the kernels' status word after the step and raise `StepError` if it is raised
        (this waits for the step; a caller that reads the word with its own results, as `Engine`
        does in the copy that brings the token ids back, passes False)."""
        spans, tables = self._reserve(entries, trusted)
        n_tokens = sum(len(e[1]) for e in entries)
        graphed = (self.use_graphs and n_tokens == len(entries) and self.graphs.bucket(len(entries)) is not None
                   and all(len(e[2]) <= 1 for e in entries))
        if device_tokens is not None and not graphed:
            raise StepError("tokens from the device need a step of single tokens on the graph path")
        if graphed:
            full = self.graphs.run(spans, tables, device_tokens)            # logits of every row
            keep = [i for i, e in enumerate(entries) if len(e[2]) == 1]
            if len(keep) == len(entries):
                logits = full
            else:
                logits = full[torch.tensor(keep, dtype=torch.long, device=self.device)] if keep else full[:0]
        else:
            logits = self.shape_graphs.run(spans, tables) if self.use_graphs else None
            if logits is None:
                spans, tables = self._pad_rows(spans, tables)
                batch = pack_step(self.ops, self.dtype, self.device, spans, tables, pin=True)
                logits = self.model.forward(batch, self.cache)
        for rid, tokens, _ in entries:
            self.processed[rid] += len(tokens)
        self.steps += 1
        self.tokens_run += n_tokens
        if check:
            self.check_status(self.steps - 1)
        return logits


def pad_rows(spans, tables, page_size: int):
    """Round a step's row count up (to a multiple of 32 up to 256 rows, of 64 beyond) with a span of
    the null request (null slot, null pages, nothing wanted), so that the library's matrix products
    see few distinct row counts: it plans every new shape once, at a millisecond each, and a
    serving run would otherwise meet thousands of them.  The added span lies at positions 0..pad-1;
    every table is widened so that its row covers them."""
    n = sum(len(s[2]) for s in spans)
    if n <= 16:                                                # the few-rows kernels: no library product
        return spans, tables
    step = 32 if n <= 256 else 64
    pad = -n % step
    if pad == 0:
        return spans, tables
    spans = list(spans) + [(None, 0, [0] * pad, [], NULL_SLOT)]
    out = {}
    for g, t in tables.items():
        m = np.asarray(t, dtype=np.int32).reshape(len(spans) - 1, -1)
        wide = np.full((len(spans), max(m.shape[1], -(-pad // page_size), 1)), NULL_PAGE, dtype=np.int32)
        wide[:len(spans) - 1, :m.shape[1]] = m
        out[g] = wide
    return spans, out


def load_runner(model_dir: str, dtype="bfloat16", max_tokens: int = 4096, max_requests: int = 64,
                page_size: int = 64, device=None, ops=None, graphs: bool = True,
                max_positions: Optional[int] = None, unexpected_tensors: str = "error") -> ModelRunner:
    """Read config.json, build the model its architecture names, load the tensors and make a cache
    for `max_tokens` positions.  `unexpected_tensors`: "error" (stored tensors that the model does not ask
    for are listed in the loader's error) or "warn" (they are passed over with a note)."""
    from ..config import load_config
    from ..weights import load_tensors
    tdtype = parse_dtype(dtype)
    if ops is None:
        from ..kernels import ops as cuda_ops
        ops = cuda_ops
        ops.require(tdtype)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if ops.device_type == "cuda" else torch.device("cpu")
    device = torch.device(device)
    cfg = load_config(model_dir)
    model = build_model(cfg)
    tensors = load_tensors(model_dir, model.param_decls(), tdtype, device, unexpected=unexpected_tensors)
    model.bind(tensors, tdtype)
    num_pages = max(-(-int(max_tokens) // page_size), 1)
    cache = CacheManager(model.cache_needs(), page_size, num_pages, max_requests, tdtype, device)
    runner = ModelRunner(model, cache, ops, tdtype, device)
    runner.config = cfg
    if graphs:
        runner.enable_graphs(min(max_positions or model.spec.max_positions, model.spec.max_positions))
    return runner


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype in (torch.bfloat16, torch.float32):
            return dtype
        raise ValueError(f"dtype {dtype} is not supported; use bfloat16 or float32")
    names = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
             "f32": torch.float32}
    if dtype not in names:
        raise ValueError(f"dtype {dtype!r} is not supported; use bfloat16 or float32")
    return names[dtype]
