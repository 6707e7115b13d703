"""Decode steps as CUDA graphs.

The reference captures one token's launches (about 290) once and replays them per token, with the
per-token scalars in pinned staging that captured copies read (src/cuda/decode_graph.zig:44-143,
`captureDecodeGraph` src/main.zig:327-403).  Here a step in which every request brings exactly one
token is captured once per batch-size bucket: the batch description lives in one fixed device
buffer that is overwritten before each replay, rows beyond the live requests point at the null
page and the null slot, and the logits come out of a fixed buffer.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.manager import NULL_PAGE, NULL_SLOT
from .batch import StepBatch

BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


class StaticDecodeStep:
    """The description of a decode batch of fixed size B in fixed device memory."""

    def __init__(self, ops, dtype, device, B: int, widths: Dict[int, int], page_size: int = 1):
        self.B, self.widths = B, dict(widths)
        n = 3 * B + (B + 1) + 3 * B + sum(B * w for w in widths.values())
        self.host = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(n, dtype=torch.int32, device=device)
        off = 0

        def take(k):
            nonlocal off
            v = (self.host[off:off + k], self.dev[off:off + k])
            off += k
            return v
        self.tok, self.pos, self.sidx = take(B), take(B), take(B)
        self.cu, self.ctx, self.slots, self.rows = take(B + 1), take(B), take(B), take(B)
        self.tables = {g: take(B * w) for g, w in widths.items()}
        self._sidx, self._cu, self._rows = list(range(B)), list(range(B + 1)), list(range(B))
        self.n_ints = n
        self.batch = StepBatch(
            ops=ops, dtype=dtype, n_tokens=B, n_seqs=B, n_wanted=B, token_ids=self.tok[1], positions=self.pos[1],
            seq_idx=self.sidx[1], cu_q=self.cu[1], ctx_lens=self.ctx[1], slot_ids=self.slots[1],
            logit_rows=self.rows[1],
            block_tables={g: self.tables[g][1].view(B, w) for g, w in widths.items()},
            max_q_len=1, max_kv_len=max(widths.values(), default=1) * page_size, decode_only=True, q_lens=[1] * B, request_ids=[None] * B)

    def pack(self, spans, tables: Dict[int, List[List[int]]], host: torch.Tensor = None) -> torch.Tensor:
        """Write the description of the live rows (request, ctx_len, [token], wanted, slot) and padding
        into a pinned host buffer (this step's own if none is given)."""
        host = self.host if host is None else host
        n, B = len(spans), self.B
        pad = B - n
        tok = [int(s[2][0]) for s in spans] + [0] * pad
        ctx = [int(s[1]) for s in spans] + [0] * pad
        slots = [int(s[4]) for s in spans] + [NULL_SLOT] * pad
        flat = tok + ctx + self._sidx + self._cu + ctx + slots + self._rows
        for g, w in self.widths.items():
            for r in tables[g]:
                flat += r[:w] if len(r) >= w else r + [NULL_PAGE] * (w - len(r))
            flat += [NULL_PAGE] * (w * pad)
        host.copy_(torch.tensor(flat, dtype=torch.int32))
        return host

    def fill(self, spans, tables: Dict[int, List[List[int]]]) -> None:
        self.upload(self.pack(spans, tables))

    def upload(self, host: torch.Tensor) -> None:
        self.dev.copy_(host, non_blocking=True)


class DecodeGraphs:
    def __init__(self, model, cache, ops, dtype, device, max_positions: int):
        self.model, self.cache, self.ops, self.dtype, self.device = model, cache, ops, dtype, device
        self.widths = {g: max(-(-max_positions // cache.page_size), 1) for g in cache.paged_groups()}
        self.graphs: Dict[int, tuple] = {}
        self.launches_per_replay: Dict[int, int] = {}
        self.replays = 0

    def bucket(self, n: int):
        for b in BUCKETS:
            if n <= b:
                return b
        return None

    def _capture(self, B: int):
        static = StaticDecodeStep(self.ops, self.dtype, self.device, B, self.widths, self.cache.page_size)
        static.fill([], {g: [] for g in self.widths})
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):                       # warm up: lazy initialisations happen outside the capture
                self.model.forward(static.batch, self.cache)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = getattr(self.ops, "launches", 0)
        with torch.cuda.graph(graph):
            logits = self.model.forward(static.batch, self.cache)
        self.launches_per_replay[B] = getattr(self.ops, "launches", 0) - before
        if hasattr(self.ops, "launches"):
            self.ops.launches = before               # captured, not run
        self.graphs[B] = (graph, static, logits)
        return self.graphs[B]

    def prepare(self, spans, tables):
        """Pack a step's description into a pinned buffer of its own, to be run later by `run_prepared`."""
        B = self.bucket(len(spans))
        _, static, _ = self.graphs.get(B) or self._capture(B)
        host = torch.empty(static.n_ints, dtype=torch.int32).pin_memory()
        return B, len(spans), static.pack(spans, tables, host)

    def run_prepared(self, prepared) -> torch.Tensor:
        B, n, host = prepared
        graph, static, logits = self.graphs[B]
        static.upload(host)
        graph.replay()
        self.replays += 1
        if hasattr(self.ops, "launches"):
            self.ops.launches += self.launches_per_replay[B]
        return logits[:n]

    def run(self, spans, tables) -> torch.Tensor:
        B = self.bucket(len(spans))
        graph, static, logits = self.graphs.get(B) or self._capture(B)
        static.fill(spans, tables)
        graph.replay()
        self.replays += 1
        if hasattr(self.ops, "launches"):
            self.ops.launches += self.launches_per_replay[B]
        return logits[:len(spans)]
