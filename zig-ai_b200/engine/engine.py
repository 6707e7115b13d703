"""Generation: requests in, tokens out.

The reference's driver (`runHybridInference`, src/main.zig:573-1417) loads the model, submits one
sequence to the scheduler, runs its prompt in chunks, samples, and loops decode steps until
`max_new_tokens` or EOS (:832-865, :990, :1138-1348), then prints prefill time and tokens per
second (:1353-1368).  `Engine` does the same for many requests at once: each `step()` asks the
scheduler for a plan, runs it through the step function, samples on the device and hands the
tokens back to the scheduler.

While every running request is decoding, the engine keeps one step ahead of the host: the next
step is launched with its input tokens still on the device (the ids the sampling kernel of the
step before wrote), and only then are that earlier step's ids read back, so planning, packing and
the read-back overlap the device's work.  A request that turns out to have ended (an EOS token) has
one row computed in vain, which is dropped.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import torch

from ..sampling.sampler import Sampler, SamplingParams
from .runner import ModelRunner, StepError, load_runner
from .scheduler import RUNNING, PlanEntry, Request, Scheduler, StepPlan


class Engine:
    def __init__(self, model_dir: str, dtype="bfloat16", max_num_seqs: int = 64, max_batched_tokens: int = 2048,
                 max_model_len: Optional[int] = None, max_tokens: Optional[int] = None, page_size: int = 64,
                 device=None, ops=None, pipeline: bool = True, profile: bool = False,
                 unexpected_tensors: str = "error"):
        """`max_tokens`: positions the cache pool holds in all (default: room for `max_num_seqs`
        requests of `max_model_len`, capped at 1 Mi positions).  `pipeline`: keep one decode step
        ahead of the host (a step's tokens are then handed out by the `step()` call after it).
        `profile`: time every step's kernels by class with CUDA events (`profile_report()`); steps are
        then launched kernel by kernel, not replayed as graphs, and none runs ahead of the host.
        `unexpected_tensors`: see `load_runner`."""
        from ..config import load_config
        cfg = load_config(model_dir)
        model_max = getattr(cfg, "max_position_embeddings", 1 << 30)
        self.max_model_len = min(int(max_model_len), model_max) if max_model_len else min(model_max, 8192)
        if max_tokens is None:
            max_tokens = min(self.max_model_len * max_num_seqs, 1 << 20)
        self.runner: ModelRunner = load_runner(model_dir, dtype, max_tokens=max_tokens, max_requests=max_num_seqs,
                                               page_size=page_size, device=device, ops=ops,
                                               max_positions=self.max_model_len, graphs=not profile,
                                               unexpected_tensors=unexpected_tensors)
        self.profile = bool(profile) and hasattr(self.runner.ops, "profile_begin")
        self._profile: Dict[str, Dict[str, float]] = {}
        self.config = self.runner.config
        self.scheduler = Scheduler(self.runner.cache, max_num_seqs, max_batched_tokens, self.max_model_len,
                                   owner=self.runner)
        self.sampler = Sampler(self.runner.ops, self.runner.device)
        self._next_id = 0
        self.pipeline = bool(pipeline) and not profile
        self._inflight = None             # a launched step not read back yet: (plan, requests in row order, ids on the
        #                                   device, their pinned host copy, the event after that copy)
        self._host_ids: List[torch.Tensor] = []
        self._host_turn = 0
        self.n_lookahead = 0
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
    def _launch(self, plan: StepPlan, device_tokens: Optional[torch.Tensor] = None):
        """Run the plan's step and its sampling kernel; nothing is read back."""
        entries = [(e.request.request_id, e.tokens, [len(e.tokens) - 1] if e.sample else []) for e in plan.entries]
        if self.profile:
            self.runner.ops.profile_begin()
        logits = self.runner.step(entries, trusted=True, device_tokens=device_tokens, check=False)
        number = self.runner.steps - 1
        wanting = [e.request for e in plan.entries if e.sample]
        ahead = 1 if device_tokens is not None else 0         # one token of each output is still on the device
        on_device = logits.device.type == "cuda"
        n = len(wanting)
        ids = self.sampler.sample_device(logits, [r.params for r in wanting], [len(r.output) + ahead for r in wanting],
                                         [r.output for r in wanting], with_status=on_device and n > 0,
                                         keys=[r.request_id for r in wanting])
        if self.profile:
            kind = "decode steps" if all(len(e.tokens) == 1 for e in plan.entries) else "steps with prompt portions"
            acc = self._profile.setdefault(kind, {"steps": 0, "tokens": 0})
            acc["steps"] += 1
            acc["tokens"] += plan.n_tokens
            for name, ms in self.runner.ops.profile_end().items():
                acc[name] = acc.get(name, 0.0) + ms
        # The kernels' status word comes with the ids: the sampling kernel put it behind them (n + 1 ints, one
        # copy); the copy to the host is queued now, before any later step's kernels, so that reading it
        # waits for this step only
        status = getattr(self.runner.ops, "status_tensor", None)
        status = status(self.runner.device) if status else None
        if not on_device:
            host = torch.cat([ids.to(torch.int32), status.to(torch.int32)]) if status is not None else ids
            if status is not None:
                status.zero_()
            return plan, wanting, ids, host, None, number
        if not self._host_ids:
            self._host_ids = [torch.empty((max(self.scheduler.max_num_seqs, 1) + 1,), dtype=torch.int32).pin_memory()
                              for _ in range(4)]
        host = self._host_ids[self._host_turn % len(self._host_ids)]
        self._host_turn += 1
        if n + 1 > host.shape[0]:
            host = torch.empty((n + 1,), dtype=torch.int32).pin_memory()
        if n > 0:
            host[:n + 1].copy_(ids, non_blocking=True)
            ids = ids[:n]
        else:
            host[:1].copy_(status, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return plan, wanting, ids, host, done, number

    def _collect(self, launched) -> List[Request]:
        """Read a launched step's token ids and hand them to the scheduler; returns the requests that ended."""
        plan, wanting, _ids_dev, host, done, number = launched
        if done is not None:
            done.synchronize()
        ids = host[:len(wanting)].tolist()
        code = int(host[len(wanting)]) if host.shape[0] > len(wanting) else 0
        if code:
            # a kernel met an id outside its bound or gave up a wait: the step's tokens are void
            ops = self.runner.ops
            if done is not None:
                ops.status_tensor(self.runner.device).zero_()
            self._inflight = None
            raise StepError(f"step {number}: {ops.describe_status(code)} (status {code}); its results are void")
        # rows of requests that ended while this step was already on its way count for nothing
        plan.entries = [e for e in plan.entries if e.request.status == RUNNING]
        sampled = {r.request_id: t for r, t in zip(wanting, ids) if r.status == RUNNING}
        self.n_steps += 1
        self.n_generated += len(sampled)
        self.n_prompt_tokens += plan.n_tokens
        return self.scheduler.commit(plan, sampled)

    def _decoding_only(self, plan: StepPlan) -> bool:
        sch = self.scheduler
        return (not sch.waiting and not plan.preempted and not plan.failed and len(plan.entries) == len(sch.running)
                and all(e.sample and len(e.tokens) == 1
                        and (e.request.params.repetition_penalty == 1.0 or self.sampler.device_history)
                        for e in plan.entries)
                and self.runner.can_take_device_tokens(len(plan.entries)))

    def _plan_ahead(self, launched) -> Optional[StepPlan]:
        """The step after `launched` (whose tokens are not known yet), if it can be planned without
        them: every request decodes on, none can end other than by an EOS token, pages are free."""
        plan = launched[0]
        if not self._decoding_only(plan) or len(plan.entries) > self.scheduler.max_batched_tokens:
            return None
        cache = self.scheduler.cache
        for e in plan.entries:
            r, p = e.request, e.request.params
            if len(r.output) + 1 >= p.max_new_tokens or len(r.prompt) + len(r.output) + 1 >= self.max_model_len:
                return None                                    # the launched step's token is its last
        for e in plan.entries:
            r = e.request
            if not cache.can_reserve(r.request_id, r.computed + 2):
                return None                                    # the scheduler decides who makes room
            cache.reserve(r.request_id, r.computed + 2)
        return StepPlan(entries=[PlanEntry(e.request, [0], True) for e in plan.entries])

    def flush(self) -> List[Request]:
        """Read back a step that is still on its way, if any; returns the requests that ended in it."""
        if self._inflight is None:
            return []
        launched, self._inflight = self._inflight, None
        return self._retire(self._collect(launched))

    def _retire(self, ended: List[Request]) -> List[Request]:
        for r in ended:
            self.requests.pop(r.request_id, None)
            self.sampler.forget(r.request_id)
        return ended

    def step(self) -> List[Request]:
        """Plan, run and sample one step; returns the requests that ended (with `pipeline`, those
        that ended in the step launched by the call before)."""
        ended: List[Request] = []
        if self._inflight is not None:
            launched, self._inflight = self._inflight, None
            plan_ahead = self._plan_ahead(launched)
            if plan_ahead is not None:
                ahead = self._launch(plan_ahead, device_tokens=launched[2])
                self.n_lookahead += 1
                ended = self._collect(launched)
                self._inflight = ahead
                return self._retire(ended)
            ended = self._collect(launched)                    # and plan the next step with its tokens known
        plan: StepPlan = self.scheduler.schedule()
        ended += plan.failed
        if plan.entries:
            launched = self._launch(plan)
            if self.pipeline and self._decoding_only(plan):
                self._inflight = launched                      # read back by the next call
            else:
                ended += self._collect(launched)
        return self._retire(ended)

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
        self.flush()                                           # a step launched ahead for requests that have ended
        failed = [done[i] for i in ids if done[i].finish_reason == "out_of_pages"]
        if failed:
            raise RuntimeError(f"{len(failed)} request(s) could not be served: out of pages")
        return [done[i].output for i in ids]

    def warm_up(self, n_seqs: int = 1) -> None:
        """What only the first steps pay (libraries' first calls, the capture of the decode graph for `n_seqs`
        requests), paid now: a request of two tokens is run to its second new token, and the graph of the bucket is
        captured from a dry run.  For a caller that wants its first request timed like the ones after it."""
        rid = self.add_request([0, 0], SamplingParams(temperature=0.0, max_new_tokens=2), request_id=("warm-up", self._next_id))
        while rid in self.requests:
            self.step()
        self.flush()
        graphs = getattr(self.runner, "graphs", None)
        if graphs is not None and getattr(self.runner, "use_graphs", False):
            bucket = graphs.bucket(max(int(n_seqs), 1))
            if bucket is not None and bucket not in graphs.graphs:
                graphs._capture(bucket)

    def profile_report(self) -> Dict[str, Dict[str, float]]:
        """With `profile=True`: per kind of step, the number of steps and tokens and the milliseconds
        its kernels took by class (the reference's PERF_STAGE table, src/main.zig:1369-1412)."""
        return {k: dict(v) for k, v in self._profile.items()}

    def stats(self) -> dict:
        out = dict(self.runner.cache.stats())
        out.update(steps=self.n_steps, generated=self.n_generated, tokens_run=self.n_prompt_tokens,
                   steps_ahead=self.n_lookahead,
                   preemptions=self.scheduler.n_preemptions, running=len(self.scheduler.running),
                   waiting=len(self.scheduler.waiting))
        return out


def generate(model_dir: str, prompts: Sequence[Sequence[int]], dtype="bfloat16", **kwargs) -> List[List[int]]:
    """One-call generation: load the model folder and generate for every prompt."""
    engine_keys = ("max_num_seqs", "max_batched_tokens", "max_model_len", "max_tokens", "page_size")
    eng = Engine(model_dir, dtype, **{k: kwargs.pop(k) for k in engine_keys if k in kwargs})
    return eng.generate(prompts, **kwargs)
