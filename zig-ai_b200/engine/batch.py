"""The description of one step's batch, as the parts and kernels see it.

A step runs, for each of S requests, a span of q_len >= 1 new tokens that starts at position
ctx_len (the tokens the cache already holds): a prompt portion, cut anywhere, or a single decoded
token.  The spans are flattened into N rows.  (The reference runs one sequence:
`forwardGPU(x, out, start_pos, n)`, src/transformer/hybrid_layer.zig:607-614.)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence

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
    scratch: Dict = field(default_factory=dict)   # what kernels compute once per step (rotation tables)


def pack_step(ops, dtype, device, spans, tables: Dict[int, List[List[int]]], pin: bool = False,
              pad_to: int = 0) -> StepBatch:
    """Build the device-side description from host lists with one host-to-device copy.
    `spans` is a list of (request_id, ctx_len, tokens, wanted offsets, slot)."""
    S = len(spans)
    tok, pos, sidx, cu, ctx, slots, rows, q_lens, rids = [], [], [], [0], [], [], [], [], []
    for s, (rid, c, tokens, want, slot) in enumerate(spans):
        n = len(tokens)
        base = len(tok)
        tok.extend(int(t) for t in tokens)
        pos.extend(range(c, c + n))
        sidx.extend([s] * n)
        cu.append(base + n)
        ctx.append(c)
        slots.append(slot)
        q_lens.append(n)
        rids.append(rid)
        for w in want:
            if not 0 <= w < n:
                raise ValueError(f"wanted place {w} is outside the {n} tokens of request {rid!r}")
            rows.append(base + w)
    N, R = len(tok), len(rows)
    parts = [tok, pos, sidx, cu, ctx, slots, rows]
    widths = {}
    for g, t in tables.items():
        widths[g] = len(t[0]) if t else 1
        parts.append([p for row in t for p in row])
    flat = [x for p in parts for x in p]
    host = torch.tensor(flat, dtype=torch.int32)
    if pin and device.type == "cuda":
        host = host.pin_memory()
    dev = host.to(device, non_blocking=True) if device.type == "cuda" else host
    off = 0
    views = []
    for p in parts:
        views.append(dev[off:off + len(p)])
        off += len(p)
    bt = {}
    for i, g in enumerate(tables):
        bt[g] = views[7 + i].view(S, widths[g]) if S else views[7 + i].view(0, 1)
    return StepBatch(
        ops=ops, dtype=dtype, n_tokens=N, n_seqs=S, n_wanted=R,
        token_ids=views[0], positions=views[1], seq_idx=views[2], cu_q=views[3], ctx_lens=views[4],
        slot_ids=views[5], logit_rows=views[6], block_tables=bt,
        max_q_len=max(q_lens) if q_lens else 0,
        max_kv_len=max((c + n for c, n in zip(ctx, q_lens)), default=0),
        decode_only=all(n == 1 for n in q_lens) and S > 0,
        q_lens=q_lens, request_ids=rids)
