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

import numpy as np
import torch

from ..cache.manager import NULL_PAGE, NULL_SLOT
from .batch import StepBatch

BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)
HOST_BUFFERS = 3        # pinned staging buffers per graph, used in turn


class StaticDecodeStep:
    """The description of a decode batch of fixed size B in fixed device memory."""

    def __init__(self, ops, dtype, device, B: int, widths: Dict[int, int], page_size: int = 1):
        self.B, self.widths = B, dict(widths)
        n = 3 * B + (B + 1) + 3 * B + sum(B * w for w in widths.values())
        # Pinned staging, taken in turn: the copy to the device is asynchronous, and a caller that keeps a
        # step ahead of the host packs the next description while the last one's copy may still be queued.
        self.hosts = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(HOST_BUFFERS)]
        self.turn = 0
        self.host = self.hosts[0]
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
        self.n_ints = n
        # layout: tok[B] pos[B] seq_idx[B] cu[B+1] ctx[B] slots[B] rows[B] tables...; constant parts and
        # padding (token 0, position 0, null slot, null page) come from a template
        t = np.zeros(n, dtype=np.int32)
        t[2 * B:3 * B] = np.arange(B)
        t[3 * B:4 * B + 1] = np.arange(B + 1)
        t[5 * B + 1:6 * B + 1] = NULL_SLOT
        t[6 * B + 1:7 * B + 1] = np.arange(B)
        t[7 * B + 1:] = NULL_PAGE
        self._template = t
        self._table_off, o = {}, 7 * B + 1
        for g, w in widths.items():
            self._table_off[g] = o
            o += B * w
        self.batch = StepBatch(
            ops=ops, dtype=dtype, n_tokens=B, n_seqs=B, n_wanted=B, token_ids=self.tok[1], positions=self.pos[1],
            seq_idx=self.sidx[1], cu_q=self.cu[1], ctx_lens=self.ctx[1], slot_ids=self.slots[1],
            logit_rows=self.rows[1],
            block_tables={g: self.tables[g][1].view(B, w) for g, w in widths.items()},
            max_q_len=1, max_kv_len=max(widths.values(), default=1) * page_size, decode_only=True, q_lens=[1] * B, request_ids=[None] * B)

    def pack(self, spans, tables, host: torch.Tensor = None) -> torch.Tensor:
        """Write the description of the live rows (request, ctx_len, [token], wanted, slot) and padding
        into a pinned host buffer (this step's own if none is given).  `tables[g]` is [n, >= width]."""
        if host is None:
            self.turn = (self.turn + 1) % len(self.hosts)
            host = self.host = self.hosts[self.turn]
        hv = host.numpy()
        n, B = len(spans), self.B
        hv[:] = self._template
        if n:
            tok = np.fromiter((s[2][0] for s in spans), dtype=np.int32, count=n)
            ctx = np.fromiter((s[1] for s in spans), dtype=np.int32, count=n)
            slots = np.fromiter((s[4] for s in spans), dtype=np.int32, count=n)
            hv[0:n] = tok
            hv[B:B + n] = ctx
            hv[4 * B + 1:4 * B + 1 + n] = ctx
            hv[5 * B + 1:5 * B + 1 + n] = slots
            for g, w in self.widths.items():
                off = self._table_off[g]
                t = np.asarray(tables[g], dtype=np.int32)
                cols = min(w, t.shape[1]) if t.ndim == 2 else 0
                if cols:
                    hv[off:off + B * w].reshape(B, w)[:n, :cols] = t[:, :cols]
        return host

    def fill(self, spans, tables: Dict[int, List[List[int]]]) -> None:
        self.upload(self.pack(spans, tables))

    def upload(self, host: torch.Tensor) -> None:
        self.dev.copy_(host, non_blocking=True)


def round_rows(n: int) -> int:
    """The row counts that steps outside the single-token graphs are rounded up to: 8, 16, then
    multiples of 32 up to 256, then multiples of 64."""
    if n <= 8:
        return 8
    if n <= 16:
        return 16
    step = 32 if n <= 256 else 64
    return -(-n // step) * step


def round_count(n: int) -> int:
    """The counts of spans and of wanted rows that a bucket is made for: 8, 16, 32, 64, then multiples
    of 64.  (Coarse on purpose: a spare span or wanted row costs next to nothing, a bucket that is
    met too rarely to be captured costs a step launched kernel by kernel.)"""
    for c in (8, 16, 32, 64):
        if n <= c:
            return c
    return -(-n // 64) * 64


class ShapeGraphs:
    """Graphs for steps that are not single-token steps (prompt portions, alone or beside decoded
    tokens).  A graph serves every step of its bucket: the row count rounded up (`round_rows`), the
    number of spans and of wanted rows rounded up (`round_count`), and the number of leading one-token
    spans rounded down to 0, 8, 16, 32, ... (attention runs those through its single-token kernel).  A step is brought to its bucket
    with a span of the null request for the spare rows (null slot and page), spans without tokens,
    and wanted rows that repeat row 0; what the kernels launch depends on those rounded counts only
    (span attention launches an upper bound of its blocks of query rows).  A bucket is captured the
    third time it is seen (a capture costs two passes and the instantiation, some tens of milliseconds
    for a full step); the most recently used graphs are kept."""

    KEEP = 16
    SEEN_BEFORE_CAPTURE = 2

    def __init__(self, model, cache, ops, dtype, device, widths: Dict[int, int]):
        self.model, self.cache, self.ops, self.dtype, self.device = model, cache, ops, dtype, device
        # the span of the null request that fills a bucket's spare rows lies at positions 0..63 at most:
        # every table row is wide enough for them, however few positions the pool holds
        self.widths = {g: max(w, -(-64 // cache.page_size)) for g, w in widths.items()}
        self.seen: Dict[tuple, int] = {}
        self.graphs: Dict[tuple, tuple] = {}          # key -> (graph, pinned staging buffers, dev, logits, launches)
        self.replays = 0

    @staticmethod
    def key(spans) -> tuple:
        n = sum(len(s[2]) for s in spans)
        r = sum(len(s[3]) for s in spans)
        from .batch import leading_singles
        return round_rows(n), round_count(len(spans) + 1), round_count(r), leading_singles([len(s[2]) for s in spans] + [0])

    def _fill(self, k, spans, tables):
        """The step in its bucket's layout: (spans, tables) with the padding spans added."""
        n_rows, n_spans = k[0], k[1]
        n = sum(len(s[2]) for s in spans)
        extra = n_spans - len(spans)
        spans = list(spans) + [(None, 0, [0] * (n_rows - n), [], NULL_SLOT)] + [(None, 0, [], [], NULL_SLOT)] * (extra - 1)
        out = {}
        for g, t in tables.items():
            m = np.asarray(t, dtype=np.int32).reshape(len(spans) - extra, -1)
            out[g] = np.vstack([m, np.full((extra, m.shape[1]), NULL_PAGE, dtype=np.int32)])
        return spans, out

    def _views(self, k, dev, lay):
        from .batch import batch_views
        batch = batch_views(self.ops, self.dtype, dev, lay)
        batch.max_kv_len = max(self.widths.values(), default=1) * self.cache.page_size
        batch.attn_tiles = k[0] // 128 + k[1]                  # every span may end with a partial block of query rows
        batch.single_first = k[3]
        return batch

    def run(self, spans, tables):
        """Logits if this step's bucket has a graph or has earned one, else None (the caller runs it eagerly)."""
        from .batch import pack_host
        k = self.key(spans)
        n_wanted = sum(len(s[3]) for s in spans)
        entry = self.graphs.get(k)
        if entry is None:
            n = self.seen.get(k, 0)
            self.seen[k] = n + 1
            if len(self.seen) > 4096:
                self.seen.clear()
            if n < self.SEEN_BEFORE_CAPTURE:
                return None
            spans_p, tables_p = self._fill(k, spans, tables)
            flat, lay = pack_host(spans_p, tables_p, self.widths, pad_wanted=k[2])
            host = torch.empty(lay.total, dtype=torch.int32).pin_memory()
            host.numpy()[:] = flat
            dev = host.to(self.device)
            batch = self._views(k, dev, lay)
            # the capture's own warm-up would run the step three times; state that a step changes in
            # place (conv state, pages) must see it once.  So this step runs eagerly now, and the
            # graph is captured from a dry run on the null request's slot and page afterwards.
            return self._capture_later(k, spans_p, tables_p, lay, host, dev, batch)[:n_wanted]
        graph, hosts, dev, logits, launches = entry
        spans_p, tables_p = self._fill(k, spans, tables)
        flat, _ = pack_host(spans_p, tables_p, self.widths, pad_wanted=k[2])
        hosts.append(hosts.pop(0))                    # staging buffers in turn (the copy below is asynchronous)
        host = hosts[0]
        host.numpy()[:] = flat
        dev.copy_(host, non_blocking=True)
        graph.replay()
        self.replays += 1
        if hasattr(self.ops, "launches"):
            self.ops.launches += launches
        self.graphs[k] = self.graphs.pop(k)           # most recently used last
        return logits[:n_wanted]

    def _capture_later(self, k, spans, tables, lay, host, dev, batch):
        from .batch import pack_host
        # dry-run description: same bucket, every span on the null slot and the null page at position 0
        dry = [(None, 0, s[2], s[3], NULL_SLOT) for s in spans]
        dry_tables = {g: np.zeros((len(spans), 1), dtype=np.int32) for g in tables}
        flat, _ = pack_host(dry, dry_tables, self.widths, pad_wanted=k[2])
        # 1. the real step, eagerly, on the static buffers
        logits_now = self.model.forward(batch, self.cache)
        # 2. capture on the dry description (the pass above was the warm-up)
        host.numpy()[:] = flat
        dev.copy_(host)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = getattr(self.ops, "launches", 0)
        with torch.cuda.graph(graph):
            logits = self.model.forward(batch, self.cache)
        launches = getattr(self.ops, "launches", 0) - before
        if hasattr(self.ops, "launches"):
            self.ops.launches = before
        while len(self.graphs) >= self.KEEP:
            self.graphs.pop(next(iter(self.graphs)))
        hosts = [host] + [torch.empty_like(host).pin_memory() for _ in range(HOST_BUFFERS - 1)]
        self.graphs[k] = (graph, hosts, dev, logits, launches)
        return logits_now


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

    def run(self, spans, tables, device_tokens: torch.Tensor = None) -> torch.Tensor:
        """`device_tokens` (int32 [rows], on the device): the rows' tokens, taken instead of the ones
        in `spans`, for a caller whose tokens are still on the device."""
        B = self.bucket(len(spans))
        graph, static, logits = self.graphs.get(B) or self._capture(B)
        static.fill(spans, tables)
        if device_tokens is not None:
            static.tok[1][:len(spans)].copy_(device_tokens)
        graph.replay()
        self.replays += 1
        if hasattr(self.ops, "launches"):
            self.ops.launches += self.launches_per_replay[B]
        return logits[:len(spans)]
