"""Plain PyTorch versions of the engine's kernels, one function per kernel with the kernel's own
signature.  Two uses: each CUDA kernel is compared with its function here (`-m gpu`), and the
engine's host logic (step function, cache, scheduler) is run on the CPU with this module standing
in for the kernels (`-m "not gpu"`).  Never used by the engine itself.

Formulas: see tests/plain_lfm2.py for the citations of the reference; these functions add only
what the cache brings (pages, block tables, state slots).
"""
from __future__ import annotations

import torch

device_type = "cpu"


def require():
    return None


fuses_norm = False      # norms run on their own here


def _f(x):
    return x.to(torch.float32)


# ---- the status word, as the kernels keep it (csrc/common.cuh: ZaiStatusBit): an id outside its bound is
# replaced by id 0 and a bit is raised; the step's results are then void.
STATUS_BITS = {1: "a bounded wait inside a kernel ran out", 2: "a token id outside the vocabulary",
               4: "a block-table entry outside the page pool", 8: "a state slot outside the slots",
               16: "a position outside its request's block-table row"}
_status = torch.zeros(1, dtype=torch.int32)


def status_tensor(device=None):
    return _status


def read_status(device=None) -> int:
    v = int(_status.item())
    _status.zero_()
    return v


def describe_status(code: int) -> str:
    return "; ".join(text for bit, text in STATUS_BITS.items() if code & bit) or f"status {code}"


def _raise(bit: int) -> None:
    _status[0] |= bit


def _checked(ids, bound: int, bit: int):
    """`ids` with every entry outside [0, bound) replaced by 0 (and the bit raised if there is one)."""
    bad = (ids < 0) | (ids >= bound)
    if bool(bad.any()):
        _raise(bit)
        ids = torch.where(bad, torch.zeros_like(ids), ids)
    return ids


def embed(ids, table):
    return _f(table[_checked(ids.long(), table.shape[0], 2)])


def add_rmsnorm(h, delta, w, eps, out_dtype):
    if delta is not None:
        h += _f(delta)
    ms = (h * h).mean(dim=-1, keepdim=True)
    return (h * torch.rsqrt(ms + eps) * _f(w)).to(out_dtype)


def linear(x, w, out_dtype=None):
    out_dtype = out_dtype or x.dtype
    if x.dtype == w.dtype and x.dtype != torch.float32 and x.device.type == "cuda":
        return (x @ w.T).to(out_dtype)
    return (_f(x) @ _f(w).T).to(out_dtype)


def linear_swiglu(x, w_gate_up, ff_dim):
    return silu_mul(linear(x, w_gate_up), ff_dim)


def silu_mul(gu, ff_dim):
    g, u = _f(gu[:, :ff_dim]), _f(gu[:, ff_dim:])
    return (g * torch.sigmoid(g) * u).to(gu.dtype)


def short_conv(bcx, conv_w, conv_b, state, step, taps, write_state=True):
    N, C3 = bcx.shape
    C = C3 // 3
    L = taps
    out = torch.empty((N, C), dtype=bcx.dtype, device=bcx.device)
    cu = step.cu_q.tolist()
    slots = _checked(step.slot_ids.long(), state.shape[0], 8).tolist()
    for s in range(step.n_seqs):
        a, b = cu[s], cu[s + 1]
        x = _f(bcx[a:b])
        u = x[:, :C] * x[:, 2 * C:]
        hist = state[slots[s]][:L - 1] if L > 1 else state[slots[s]][:0]
        full = torch.cat([hist, u], dim=0)                        # [(L-1)+n, C]
        y = torch.zeros_like(u)
        for j in range(L):
            y += full[j:j + (b - a)] * conv_w[:, j][None, :]
        if conv_b is not None:
            y += conv_b[None, :]
        out[a:b] = (x[:, C:2 * C] * y).to(bcx.dtype)
        if write_state and L > 1:
            state[slots[s]][:L - 1] = full[full.shape[0] - (L - 1):]
    return out


def linear_short_conv(x, w_in, conv_w, conv_b, state, step, taps, write_state=True):
    return short_conv(linear(x, w_in), conv_w, conv_b, state, step, taps, write_state)


def _rms(x, w, eps):
    ms = (x * x).mean(dim=-1, keepdim=True)
    y = x * torch.rsqrt(ms + eps)
    return y * w if w is not None else y


def _rotate(x, positions, rotary_dim, theta):
    if rotary_dim == 0:
        return x
    half = rotary_dim // 2
    i = torch.arange(half, dtype=torch.float32, device=x.device)
    freq = torch.exp(-(2.0 * i / rotary_dim) * torch.log(torch.tensor(float(theta))))
    ang = positions.to(torch.float32)[:, None] * freq[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:rotary_dim]
    out = x.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:rotary_dim] = a * sin + b * cos
    return out


def _page_rows(step, cache):
    """For every row of the step: (page id, offset inside the page)."""
    ps = cache.page_size
    pos = step.positions.long()
    bt = cache.block_table.long()
    idx = pos // ps
    outside = (idx < 0) | (idx >= bt.shape[1])
    if bool(outside.any()):
        _raise(16)
    page = bt[step.seq_idx.long(), torch.where(outside, torch.zeros_like(idx), idx)]
    page = torch.where(outside, torch.zeros_like(page), _checked(page, cache.pages.shape[0], 4))
    return page, pos % ps


def qk_norm_rope(qkv, q_w, k_w, eps, rotary_dim, theta, step, cache, heads, kv_heads, head_dim,
                 has_kv=True, write=True, return_k=False):
    N = qkv.shape[0]
    D = head_dim
    q = _f(qkv[:, :heads * D]).reshape(N, heads, D)
    if q_w is not None:
        q = _rms(q, q_w, eps)
    q = _rotate(q, step.positions, rotary_dim, theta).to(qkv.dtype).reshape(N, heads * D)
    k_out = None
    if has_kv:
        k = _f(qkv[:, heads * D:(heads + kv_heads) * D]).reshape(N, kv_heads, D)
        if k_w is not None:
            k = _rms(k, k_w, eps)
        k = _rotate(k, step.positions, rotary_dim, theta).to(qkv.dtype)
        v = qkv[:, (heads + kv_heads) * D:].reshape(N, kv_heads, D)
        if write:
            page, off = _page_rows(step, cache)
            cache.pages[page, 0, :, off, :] = k.to(cache.pages.dtype)
            cache.pages[page, 1, :, off, :] = v.to(cache.pages.dtype)
        if return_k:
            k_out = k.reshape(N, kv_heads * D)
    return q, k_out


def kv_write(k, v, step, cache, kv_heads, head_dim):
    N = k.shape[0]
    page, off = _page_rows(step, cache)
    cache.pages[page, 0, :, off, :] = k.reshape(N, kv_heads, head_dim).to(cache.pages.dtype)
    cache.pages[page, 1, :, off, :] = v.reshape(N, kv_heads, head_dim).to(cache.pages.dtype)


def paged_attention(q, step, cache, heads, kv_heads, head_dim, scale, window=None):
    N = q.shape[0]
    D, ps = head_dim, cache.page_size
    out = torch.empty((N, heads * D), dtype=q.dtype, device=q.device)
    cu, ctx = step.cu_q.tolist(), step.ctx_lens.tolist()
    group = heads // kv_heads
    for s in range(step.n_seqs):
        a, b = cu[s], cu[s + 1]
        total = ctx[s] + (b - a)
        n_pages = -(-total // ps)
        if n_pages > cache.block_table.shape[1]:
            _raise(16)
        ids = _checked(cache.block_table[s, :n_pages].long(), cache.pages.shape[0], 4)
        ids = torch.cat([ids, ids.new_zeros(n_pages - ids.shape[0])])
        kv = _f(cache.pages[ids])                                  # [pages, 2, Hkv, ps, D]
        k = kv[:, 0].permute(1, 0, 2, 3).reshape(kv_heads, n_pages * ps, D)[:, :total]
        v = kv[:, 1].permute(1, 0, 2, 3).reshape(kv_heads, n_pages * ps, D)[:, :total]
        qs = _f(q[a:b]).reshape(b - a, heads, D).permute(1, 0, 2)   # [Hq, n, D]
        k = k.repeat_interleave(group, dim=0)
        v = v.repeat_interleave(group, dim=0)
        sc = torch.einsum("hnd,hkd->hnk", qs, k) * scale
        qpos = torch.arange(ctx[s], total, device=q.device)[:, None]
        kpos = torch.arange(total, device=q.device)[None, :]
        mask = kpos > qpos
        if window is not None:
            mask = mask | (kpos <= qpos - window)
        sc = sc.masked_fill(mask[None], float("-inf"))
        p = torch.softmax(sc, dim=-1)
        o = torch.einsum("hnk,hkd->hnd", p, v).permute(1, 0, 2).reshape(b - a, heads * D)
        out[a:b] = o.to(q.dtype)
    return out


def gather_add(h, pending, rows):
    r = rows.long()
    out = h[r].clone()
    if pending is not None:
        out += _f(pending[r])
    return out


def argmax(logits):
    """First index of the maximum of each row."""
    m = logits.max(dim=-1, keepdim=True).values
    V = logits.shape[-1]
    idx = torch.arange(V, device=logits.device)[None, :].expand_as(logits)
    return torch.where(logits == m, idx, V).min(dim=-1).values.to(torch.int32)


def sample(logits, temperature, top_k, top_p, u):
    """Row-wise sampling with given uniforms: temperature <= 0 is greedy; otherwise logits/T,
    top-k (values >= the k-th largest), top-p (shortest descending prefix reaching p), then the
    inverse CDF in index order over the kept set."""
    R, V = logits.shape
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    for r in range(R):
        T = float(temperature[r])
        if T <= 0:
            out[r] = argmax(logits[r:r + 1])[0]
            continue
        w = logits[r].to(torch.float64) / T
        k = int(top_k[r])
        if 0 < k < V:
            kth = torch.sort(w, descending=True).values[k - 1]
            w = torch.where(w >= kth, w, torch.tensor(float("-inf"), dtype=torch.float64, device=w.device))
        p = torch.softmax(w, dim=-1)
        tp = float(top_p[r])
        if tp < 1.0:
            sp, si = torch.sort(p, descending=True, stable=True)
            cum = torch.cumsum(sp, 0)
            cutoff = int((cum >= tp).nonzero()[0]) + 1 if bool((cum >= tp).any()) else V
            thresh = sp[cutoff - 1]
            p = torch.where(p >= thresh, p, torch.zeros_like(p))
        c = torch.cumsum(p, 0)
        target = float(u[r]) * float(c[-1])
        hit = (c >= target).nonzero()
        out[r] = int(hit[0]) if hit.numel() else V - 1
    return out


def repetition_penalty(logits, tokens, counts, offsets, penalty):
    off = offsets.tolist()
    for r in range(logits.shape[0]):
        p = float(penalty[r])
        for i in range(off[r], off[r + 1]):
            t = int(tokens[i])
            for _ in range(int(counts[i])):
                v = logits[r, t]
                logits[r, t] = v / p if v > 0 else (v * p if v < 0 else v)
    return logits
