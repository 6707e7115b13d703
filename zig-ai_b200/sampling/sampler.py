"""Sampling parameters, the per-request random numbers and the batched call of the sampling kernels.

The reference's sampler (src/transformer/pipeline.zig:17-151) has a temperature (<= 0 is greedy),
top-k (0 is off), top-p (1.0 is off) and a repetition penalty (1.0 is off) and draws from one
Xoshiro256 stream seeded by `--seed` (src/main.zig:760).  Here every sampled token gets its own
uniform number from a counter-based generator keyed by the request's seed and the index of the
token in the request's output, so a request's tokens do not depend on what else is in the batch,
on how its prompt was cut, or on whether it was preempted and recomputed.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

_MASK = (1 << 64) - 1


@dataclass
class SamplingParams:
    temperature: float = 1.0            # <= 0: greedy
    top_k: int = 0                      # 0: off
    top_p: float = 1.0                  # 1.0: off
    repetition_penalty: float = 1.0     # 1.0: off
    seed: int = 42
    max_new_tokens: int = 128
    eos_id: Optional[int] = None

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k should be 0 (off) or positive")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p should be in (0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty should be positive")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens should be at least 1")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, index: int) -> float:
    """A number in [0, 1) with 24 random bits (exact in 32-bit), fixed by (seed, index)."""
    z = _splitmix64(_splitmix64(seed & _MASK) ^ ((index * 0xD6E8FEB86659FD93) & _MASK))
    return (z >> 40) / float(1 << 24)


def uniforms(seeds, indices):
    """`uniform` for arrays of seeds and indices (the same numbers, computed with 64-bit array arithmetic)."""
    import numpy as np

    def mix(x):
        x = x + np.uint64(0x9E3779B97F4A7C15)
        z = x
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))

    with np.errstate(over="ignore"):
        s = np.asarray([v & _MASK for v in seeds], dtype=np.uint64)
        i = np.asarray(indices, dtype=np.uint64)
        z = mix(mix(s) ^ (i * np.uint64(0xD6E8FEB86659FD93)))
    return ((z >> np.uint64(40)).astype(np.float64) / float(1 << 24)).astype(np.float32)


class _Staging:
    """A step's small arrays on their way to the device: written into one pinned buffer and sent with one copy
    that nothing waits for (a tensor made from a Python list is copied from pageable memory, and that copy
    waits for the stream, which ends the engine's running ahead).  Buffers take turns, so a step's copy is
    long over when its buffer is written again."""

    TURNS = 4

    def __init__(self, device):
        self.device = device
        self.host: List[Optional[torch.Tensor]] = [None] * self.TURNS
        self.dev: List[Optional[torch.Tensor]] = [None] * self.TURNS
        self.turn = 0

    def send(self, parts):
        """`parts`: arrays of 32-bit numbers (float32 or int32).  Returns their device tensors."""
        import numpy as np
        n = sum(int(p.size) for p in parts)
        t = self.turn
        self.turn = (t + 1) % self.TURNS
        if self.host[t] is None or self.host[t].numel() < n:
            cap = max(1024, 2 * n)
            self.host[t] = torch.empty((cap,), dtype=torch.int32).pin_memory()
            self.dev[t] = torch.empty((cap,), dtype=torch.int32, device=self.device)
        host, dev = self.host[t], self.dev[t]
        hn = host.numpy()
        out, at = [], 0
        for p in parts:
            m = int(p.size)
            hn[at:at + m] = np.ascontiguousarray(p).view(np.int32)
            out.append((at, m, torch.float32 if p.dtype == np.float32 else torch.int32))
            at += m
        dev[:n].copy_(host[:n], non_blocking=True)
        return [dev[a:a + m].view(dt) for a, m, dt in out]


class _History:
    """The distinct tokens of one request's output and how often each came, kept up as the output grows."""

    def __init__(self):
        import numpy as np
        self.where = {}
        self.tokens = np.zeros((64,), dtype=np.int32)
        self.counts = np.zeros((64,), dtype=np.int32)
        self.n = 0
        self.seen = 0

    def update(self, output):
        import numpy as np
        if self.seen > len(output):                          # not the list this was built from: start over
            self.where, self.n, self.seen = {}, 0, 0
        for t in output[self.seen:]:
            j = self.where.get(t)
            if j is None:
                if self.n == self.tokens.shape[0]:
                    self.tokens = np.concatenate([self.tokens, np.zeros_like(self.tokens)])
                    self.counts = np.concatenate([self.counts, np.zeros_like(self.counts)])
                j = self.where[t] = self.n
                self.tokens[j] = t
                self.counts[j] = 0
                self.n += 1
            self.counts[j] += 1
        self.seen = len(output)


class Sampler:
    """Turns the logits of one step into token ids on the device, one row per request."""

    def __init__(self, ops, device):
        self.ops, self.device = ops, device
        self._staging: Optional[_Staging] = None
        self._histories = {}
        # with kernels that keep the histories on the device: a table of counts [slots, vocabulary] and the
        # slot of every request that has a repetition penalty
        self.device_history = (torch.device(device).type == "cuda" and hasattr(ops, "repetition_penalty_counts")
                               and hasattr(ops, "count_tokens"))
        self._counts: Optional[torch.Tensor] = None
        self._slots = {}
        self._free_slots: List[int] = []

    def forget(self, key) -> None:
        """The request of this name has ended: what was kept of its history is given up."""
        self._histories.pop(key, None)
        slot = self._slots.pop(key, None)
        if slot is not None:
            self._free_slots.append(slot)

    def _slot_of(self, key, history, vocab: int, live) -> int:
        """The request's row in the table of counts; a new one starts from the history it brings (empty as a rule)."""
        slot = self._slots.get(key)
        if slot is not None:
            return slot
        if not self._free_slots:
            for k in [k for k in self._slots if k not in live]:     # requests that ended without a word
                self.forget(k)
        if not self._free_slots:
            old = 0 if self._counts is None else self._counts.shape[0]
            grown = torch.zeros((max(2 * old, 16), vocab), dtype=torch.int32, device=self.device)
            if old:
                grown[:old].copy_(self._counts)
            self._counts = grown
            self._free_slots = list(range(grown.shape[0] - 1, old - 1, -1))
        slot = self._free_slots.pop()
        self._slots[key] = slot
        self._counts[slot].zero_()
        if history:
            toks = torch.tensor([t for t in history if 0 <= t < vocab], dtype=torch.long, device=self.device)
            self._counts[slot].index_put_((toks,), torch.ones_like(toks, dtype=torch.int32), accumulate=True)
        return slot

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], indices: Sequence[int],
               histories: Sequence[Sequence[int]]) -> List[int]:
        """`indices[r]` is the index of the token being sampled in row r's output; `histories[r]`
        the tokens generated so far (used by the repetition penalty only)."""
        if logits.shape[0] == 0:
            return []
        return self.sample_device(logits, params, indices, histories).tolist()

    def sample_device(self, logits: torch.Tensor, params: Sequence[SamplingParams], indices: Sequence[int],
                      histories: Sequence[Sequence[int]], with_status: bool = False, keys: Optional[Sequence] = None) -> torch.Tensor:
        """As `sample`, but the token ids stay on the device (int32 [rows]); nothing waits for them.
        `with_status` (kernels that keep a status word only): [rows + 1], the status word behind the ids.
        `keys`: a name for each row's request, under which what is known of its history is kept between calls."""
        import numpy as np
        R = logits.shape[0]
        if R == 0:
            return torch.empty((0,), dtype=torch.int32, device=self.device)
        on_cuda = logits.device.type == "cuda"
        if on_cuda and self._staging is None:
            self._staging = _Staging(self.device)

        def to_device(parts):
            if on_cuda:
                return self._staging.send(parts)
            return [torch.from_numpy(np.ascontiguousarray(p)).to(self.device) for p in parts]

        penalised = any(p.repetition_penalty != 1.0 for p in params)
        slots_dev = None
        if penalised and on_cuda and self.device_history and keys is not None:
            # the histories live on the device: the penalty reads the requests' rows of the table of counts, and
            # the tokens sampled below are counted there, so nothing of this waits for a token to reach the host
            live = set(keys)
            slots = [self._slot_of(k, h, logits.shape[1], live) if p.repetition_penalty != 1.0 else -1
                     for k, p, h in zip(keys, params, histories)]
            slots_dev, pen = to_device([np.asarray(slots, dtype=np.int32),
                                        np.asarray([p.repetition_penalty for p in params], dtype=np.float32)])
            logits = self.ops.repetition_penalty_counts(logits, self._counts, slots_dev, pen)
        elif penalised:
            toks, counts, offsets = [], [], [0]
            for r, (p, hist) in enumerate(zip(params, histories)):
                if p.repetition_penalty != 1.0:
                    key = keys[r] if keys is not None else None
                    h = self._histories.get(key) if key is not None else None
                    if h is None:
                        h = _History()
                        if key is not None:
                            self._histories[key] = h
                    h.update(hist)
                    toks.append(h.tokens[:h.n])
                    counts.append(h.counts[:h.n])
                    offsets.append(offsets[-1] + h.n)
                else:
                    offsets.append(offsets[-1])
            if keys is not None and len(self._histories) > 2 * len(keys) + 64:
                live = set(keys)
                self._histories = {k: v for k, v in self._histories.items() if k in live}
            if offsets[-1]:
                t, c, o, pen = to_device([np.concatenate(toks), np.concatenate(counts), np.asarray(offsets, dtype=np.int32),
                                          np.asarray([p.repetition_penalty for p in params], dtype=np.float32)])
                logits = self.ops.repetition_penalty(logits.clone(), t, c, o, pen)
        extra = {"with_status": True} if with_status else {}
        if all(p.greedy for p in params):
            ids = self.ops.argmax(logits, **extra)
        else:
            temperature, top_k, top_p, u = to_device([
                np.asarray([p.temperature for p in params], dtype=np.float32),
                np.asarray([p.top_k for p in params], dtype=np.int32),
                np.asarray([p.top_p for p in params], dtype=np.float32),
                uniforms([p.seed for p in params], indices)])
            ids = self.ops.sample(logits, temperature, top_k, top_p, u, **extra)
        if slots_dev is not None:
            self.ops.count_tokens(self._counts, ids, slots_dev, R)
        return ids
