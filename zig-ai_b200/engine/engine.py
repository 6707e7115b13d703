"""Generation: requests in, tokens out.

The reference's driver (`runHybridInference`, src/main.zig:573-1417) loads the model, submits one
sequence to the scheduler, runs its prompt in chunks, samples, and loops decode steps until
`max_new_tokens` or EOS (:832-865, :990, :1138-1348), then prints prefill time and tokens per
second (:1353-1368).  `Engine` does the same for many requests at once: each `step()` asks the
scheduler for a plan, runs it through the step function, samples on the device and hands the
tokens back to the scheduler.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import torch

from ..sampling.sampler import Sampler, SamplingParams
from .runner import ModelRunner, load_runner
from .scheduler import Request, Scheduler, StepPlan


class Engine:
    def __init__(self, model_dir: str, dtype="bfloat16", max_num_seqs: int = 64, max_batched_tokens: int = 2048,
                 max_model_len: Optional[int] = None, max_tokens: Optional[int] = None, page_size: int = 64,
                 device=None, ops=None):
        """`max_tokens`: positions the cache pool holds in all (default: room for `max_num_seqs`
        requests of `max_model_len`, capped at 1 Mi positions)."""
        from ..config import load_config
        cfg = load_config(model_dir)
        model_max = getattr(cfg, "max_position_embeddings", 1 << 30)
        self.max_model_len = min(int(max_model_len), model_max) if max_model_len else min(model_max, 8192)
        if max_tokens is None:
            max_tokens = min(self.max_model_len * max_num_seqs, 1 << 20)
        self.runner: ModelRunner = load_runner(model_dir, dtype, max_tokens=max_tokens, max_requests=max_num_seqs,
                                               page_size=page_size, device=device, ops=ops,
                                               max_positions=self.max_model_len)
        self.config = self.runner.config
        self.scheduler = Scheduler(self.runner.cache, max_num_seqs, max_batched_tokens, self.max_model_len,
                                   owner=self.runner)
        self.sampler = Sampler(self.runner.ops, self.runner.device)
        self._next_id = 0
        self.requests: Dict[object, Request] = {}
        self.n_steps = 0
        self.n_prompt_tokens = 0
        self.n_generated = 0

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, request_id=None):
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        if request_id in self.requests:
            raise ValueError(f"request id {request_id!r} is in use")
        V = self.runner.model.vocab_size
        bad = [int(t) for t in prompt if not 0 <= int(t) < V]
        if bad:
            raise ValueError(f"token ids {bad[:8]} are outside the vocabulary of {V}")
        req = Request(request_id, [int(t) for t in prompt], params or SamplingParams())
        self.scheduler.add(req)
        self.requests[request_id] = req
        return request_id

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    # ------------------------------------------------------------------ one step
    def step(self) -> List[Request]:
        """Plan, run and sample one step; returns the requests that ended in it."""
        plan: StepPlan = self.scheduler.schedule()
        ended = list(plan.failed)
        if plan.entries:
            entries = [(e.request.request_id, e.tokens, [len(e.tokens) - 1] if e.sample else []) for e in plan.entries]
            logits = self.runner.step(entries, trusted=True)
            wanting = [e.request for e in plan.entries if e.sample]
            ids = self.sampler.sample(logits, [r.params for r in wanting], [len(r.output) for r in wanting],
                                      [r.output for r in wanting])
            sampled = {r.request_id: t for r, t in zip(wanting, ids)}
            self.n_steps += 1
            self.n_generated += len(ids)
            self.n_prompt_tokens += plan.n_tokens
            ended += self.scheduler.commit(plan, sampled)
        for r in ended:
            self.requests.pop(r.request_id, None)
        return ended

    # ------------------------------------------------------------------ whole generation
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 128, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, repetition_penalty: float = 1.0, seed: int = 42,
                 eos_id: Optional[int] = None) -> List[List[int]]:
        """Generated token ids for every prompt (host lists in, host lists out).  Prompt i samples
        with the seed `seed + i`."""
        ids = []
        for i, p in enumerate(prompts):
            ids.append(self.add_request(p, SamplingParams(
                temperature=temperature, top_k=top_k, top_p=top_p, repetition_penalty=repetition_penalty,
                seed=seed + i, max_new_tokens=max_new_tokens, eos_id=eos_id)))
        done: Dict[object, Request] = {}
        while len(done) < len(ids):
            for r in self.step():
                done[r.request_id] = r
            if not self.has_work() and len(done) < len(ids):
                raise RuntimeError("the scheduler stopped with requests unfinished")
        failed = [done[i] for i in ids if done[i].finish_reason == "out_of_pages"]
        if failed:
            raise RuntimeError(f"{len(failed)} request(s) could not be served: out of pages")
        return [done[i].output for i in ids]

    def stats(self) -> dict:
        out = dict(self.runner.cache.stats())
        out.update(steps=self.n_steps, generated=self.n_generated, tokens_run=self.n_prompt_tokens,
                   preemptions=self.scheduler.n_preemptions, running=len(self.scheduler.running),
                   waiting=len(self.scheduler.waiting))
        return out


def generate(model_dir: str, prompts: Sequence[Sequence[int]], dtype="bfloat16", **kwargs) -> List[List[int]]:
    """One-call generation: load the model folder and generate for every prompt."""
    engine_keys = ("max_num_seqs", "max_batched_tokens", "max_model_len", "max_tokens", "page_size")
    eng = Engine(model_dir, dtype, **{k: kwargs.pop(k) for k in engine_keys if k in kwargs})
    return eng.generate(prompts, **kwargs)
