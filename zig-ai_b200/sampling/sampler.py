"""Sampling parameters, the per-request random numbers and the batched call of the sampling kernels.

The reference's sampler (src/transformer/pipeline.zig:17-151) has a temperature (<= 0 is greedy),
top-k (0 is off), top-p (1.0 is off) and a repetition penalty (1.0 is off) and draws from one
Xoshiro256 stream seeded by `--seed` (src/main.zig:760).  Here every sampled token gets its own
uniform number from a counter-based generator keyed by the request's seed and the index of the
token in the request's output, so a request's tokens do not depend on what else is in the batch,
on how its prompt was cut, or on whether it was preempted and recomputed.
"""
from __future__ import annotations

from collections import Counter
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


class Sampler:
    """Turns the logits of one step into token ids on the device, one row per request."""

    def __init__(self, ops, device):
        self.ops, self.device = ops, device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], indices: Sequence[int],
               histories: Sequence[Sequence[int]]) -> List[int]:
        """`indices[r]` is the index of the token being sampled in row r's output; `histories[r]`
        the tokens generated so far (used by the repetition penalty only)."""
        if logits.shape[0] == 0:
            return []
        return self.sample_device(logits, params, indices, histories).tolist()

    def sample_device(self, logits: torch.Tensor, params: Sequence[SamplingParams], indices: Sequence[int],
                      histories: Sequence[Sequence[int]], with_status: bool = False) -> torch.Tensor:
        """As `sample`, but the token ids stay on the device (int32 [rows]); nothing waits for them.
        `with_status` (kernels that keep a status word only): [rows + 1], the status word behind the ids."""
        R = logits.shape[0]
        if R == 0:
            return torch.empty((0,), dtype=torch.int32, device=self.device)
        if any(p.repetition_penalty != 1.0 for p in params):
            toks, counts, offsets, pens = [], [], [0], []
            for p, hist in zip(params, histories):
                if p.repetition_penalty != 1.0:
                    for t, c in Counter(hist).items():
                        toks.append(int(t))
                        counts.append(int(c))
                offsets.append(len(toks))
                pens.append(float(p.repetition_penalty))
            if toks:
                dev = self.device
                logits = self.ops.repetition_penalty(
                    logits.clone(), torch.tensor(toks, dtype=torch.int32, device=dev),
                    torch.tensor(counts, dtype=torch.int32, device=dev),
                    torch.tensor(offsets, dtype=torch.int32, device=dev),
                    torch.tensor(pens, dtype=torch.float32, device=dev))
        extra = {"with_status": True} if with_status else {}
        if all(p.greedy for p in params):
            ids = self.ops.argmax(logits, **extra)
        else:
            dev = self.device
            temperature = torch.tensor([p.temperature for p in params], dtype=torch.float32, device=dev)
            top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32, device=dev)
            top_p = torch.tensor([p.top_p for p in params], dtype=torch.float32, device=dev)
            u = torch.tensor([uniform(p.seed, i) for p, i in zip(params, indices)], dtype=torch.float32, device=dev)
            ids = self.ops.sample(logits, temperature, top_k, top_p, u, **extra)
        return ids
