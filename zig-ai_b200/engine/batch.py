"""The description of one step's batch, as the parts and kernels see it.

A step runs, for each of S requests, a span of q_len >= 1 new tokens that starts at position
ctx_len (the tokens the cache already holds): a prompt portion, cut anywhere, or a single decoded
token.  The spans are flattened into N rows.  (The reference runs one sequence:
`forwardGPU(x, out, start_pos, n)`, src/transformer/hybrid_layer.zig:607-614.)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepBatch:
    ops: object
    dtype: torch.dtype
    n_tokens: int
    n_seqs: int
    n_wanted: int
    token_ids: torch.Tensor        # [N] int32
    positions: torch.Tensor        # [N] int32, absolute position in the request
    seq_idx: torch.Tensor          # [N] int32, which of the step's requests a row belongs to
    cu_q: torch.Tensor             # [S+1] int32, first row of each request's span
    ctx_lens: torch.Tensor         # [S] int32, tokens cached before this step
    slot_ids: torch.Tensor         # [S] int32
    logit_rows: torch.Tensor       # [R] int32, rows whose logits are wanted
    block_tables: Dict[int, torch.Tensor] = field(default_factory=dict)   # group -> [S, width] int32
    max_q_len: int = 1
    max_kv_len: int = 1            # largest ctx_len + q_len
    decode_only: bool = False      # every span is one token
    q_lens: Sequence[int] = ()
    request_ids: Sequence = ()
    single_first: int = 0          # this many leading spans (0, 8, 16, 32, ...) are one token each: in a step that also
    #                                holds longer spans, attention may run them through the kernel for single tokens
    attn_tiles: Optional[int] = None   # blocks of query rows to launch for span attention (default: from q_lens);
    #                                    a captured graph launches an upper bound for its bucket of step shapes
    scratch: Dict = field(default_factory=dict)   # what kernels compute once per step (rotation tables)


@dataclass
class PackedLayout:
    """Where the pieces of a packed step lie in its flat int32 buffer."""
    N: int
    S: int
    R: int
    tables: Dict[int, tuple]           # group -> (offset, width)
    total: int
    q_lens: List[int]
    ctx: List[int]
    request_ids: List


def pack_host(spans, tables: Dict[int, "np.ndarray"], widths: Dict[int, int] = None, pad_wanted: int = 0):
    """Flatten a step's description into one int32 array: tokens, positions, row->request, span
    starts, context lengths, slots, wanted rows, then each group's block tables [S, width].  (A span
    may have no tokens.)
    `spans` is a list of (request_id, ctx_len, tokens, wanted offsets, slot); `widths` fixes the
    table widths (a captured graph needs them constant), default: as wide as the tables given."""
    S = len(spans)
    ctx, slots, rows, q_lens, rids = [], [], [], [], []
    single_at, single_tok, longer = [], [], []     # one-token spans are gathered and written in one go
    at = 0
    for rid, c, tokens, want, slot in spans:
        n = len(tokens)
        if n == 1:
            single_at.append(at)
            single_tok.append(tokens[0])
        elif n:
            longer.append((at, tokens))
        ctx.append(c)
        slots.append(slot)
        q_lens.append(n)
        rids.append(rid)
        for w in want:
            if not 0 <= w < n:
                raise ValueError(f"wanted place {w} is outside the {n} tokens of request {rid!r}")
            rows.append(at + w)
        at += n
    tok_all = np.empty(at, dtype=np.int32)
    if single_at:
        tok_all[single_at] = single_tok
    for a0, tokens in longer:
        tok_all[a0:a0 + len(tokens)] = tokens
    # positions and the rows' requests for all spans at once: row i of span s lies at ctx[s] + i
    lens = np.asarray(q_lens, dtype=np.int64)
    starts = np.zeros(S + 1, dtype=np.int64)
    np.cumsum(lens, out=starts[1:])
    sidx_all = np.repeat(np.arange(S, dtype=np.int32), lens)
    pos_all = (np.arange(at, dtype=np.int64) - np.repeat(starts[:-1], lens) + np.repeat(np.asarray(ctx, dtype=np.int64), lens)).astype(np.int32)
    tok = [tok_all] if at else []
    pos, sidx = ([pos_all], [sidx_all]) if at else ([], [])
    cu = starts.tolist()
    rows += [0] * max(pad_wanted - len(rows), 0)              # (`pad_wanted`: the wanted rows are filled up with row 0)
    parts = tok + pos + sidx + [np.array(cu + ctx + slots + rows, dtype=np.int32)]
    N, R = at, len(rows)
    off = 3 * N + (S + 1) + 2 * S + R
    layout_tables = {}
    for g, t in tables.items():
        m = np.asarray(t, dtype=np.int32).reshape(S, -1)
        w = widths[g] if widths else max(m.shape[1], 1)
        if m.shape[1] != w:
            fixed = np.zeros((S, w), dtype=np.int32)
            cols = min(w, m.shape[1])
            fixed[:, :cols] = m[:, :cols]
            m = fixed
        parts.append(m.reshape(-1))
        layout_tables[g] = (off, w)
        off += S * w
    flat = np.concatenate(parts) if parts else np.zeros(0, np.int32)
    return flat, PackedLayout(N, S, R, layout_tables, off, q_lens, ctx, rids)


def leading_singles(q_lens) -> int:
    """How many spans at the front of a step are one token each, rounded down to 8, 16, 32, 64, ...
    (0 below 8: few values, since a step's graph is made for one of them); 0 if that is all of the
    spans (a step of single tokens has its own path)."""
    n = 0
    for q in q_lens:
        if q != 1:
            break
        n += 1
    if n == len(q_lens) or n < 8:
        return 0
    return 1 << (n.bit_length() - 1)


def batch_views(ops, dtype, dev: torch.Tensor, lay: PackedLayout) -> StepBatch:
    """A StepBatch whose tensors are views of the flat device buffer `dev`."""
    N, S, R = lay.N, lay.S, lay.R
    sizes = [N, N, N, S + 1, S, S, R]
    views, at = [], 0
    for n in sizes:
        views.append(dev[at:at + n])
        at += n
    bt = {g: (dev[o:o + S * w].view(S, w) if S else dev[o:o].view(0, 1)) for g, (o, w) in lay.tables.items()}
    return StepBatch(
        single_first=leading_singles(lay.q_lens), ops=ops, dtype=dtype, n_tokens=N, n_seqs=S, n_wanted=R,
        token_ids=views[0], positions=views[1], seq_idx=views[2], cu_q=views[3], ctx_lens=views[4],
        slot_ids=views[5], logit_rows=views[6], block_tables=bt,
        max_q_len=max(lay.q_lens) if lay.q_lens else 0,
        max_kv_len=max((c + n for c, n in zip(lay.ctx, lay.q_lens)), default=0),
        decode_only=all(n == 1 for n in lay.q_lens) and S > 0,
        q_lens=lay.q_lens, request_ids=lay.request_ids)


def pack_step(ops, dtype, device, spans, tables: Dict[int, "np.ndarray"], pin: bool = False) -> StepBatch:
    """Build the device-side description from host data with one host-to-device copy."""
    flat, lay = pack_host(spans, tables)
    host = torch.empty(lay.total, dtype=torch.int32, pin_memory=bool(pin and device.type == "cuda"))
    host.numpy()[:] = flat
    dev = host.to(device, non_blocking=True) if device.type == "cuda" else host
    return batch_views(ops, dtype, dev, lay)
