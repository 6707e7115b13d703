#!/usr/bin/env python3
"""Benchmark: decode tokens per second of the LFM2-350M shape on one B200, with prefill, roofline
and end-to-end figures on the same JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 requests whose contexts lie between 2048 and 4096
tokens; weights are random (seeded), token ids are random: there is no dataset.  `value` times the
step function and the sampling kernel on the device with CUDA events; `e2e` times the same steps
through `Engine.step()`, the call a user makes, with host token lists in and out.  The decode step
reads about 0.7 GB of weights, more than the 126 MB L2, so consecutive steps cannot be served from L2.
"""
import argparse
import json
import os
import random
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LFM2_350M = {
    "architectures": ["Lfm2ForCausalLM"], "hidden_size": 1024, "num_hidden_layers": 16,
    "full_attn_idxs": [2, 5, 8, 10, 12, 14], "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 64,
    "block_ff_dim": 6656, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256, "vocab_size": 65536,
    "rope_theta": 1000000.0, "conv_L_cache": 3, "conv_bias": False, "use_qk_norm": True, "norm_eps": 1e-5,
    "tie_embedding": True, "max_position_embeddings": 128000,
}
SHAPES = {
    "350m": dict(hidden_size=1024, num_attention_heads=16, block_ff_dim=6656),
    "700m": dict(hidden_size=1536, num_attention_heads=24, block_ff_dim=10752),
    "1.2b": dict(hidden_size=2048, num_attention_heads=32, block_ff_dim=12288),
}
CONTEXT = 4096
PREFILL_TOKENS = 2048


def shape_config(name):
    d = dict(LFM2_350M)
    d.update(SHAPES[name])
    return d


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, flops, src = 6650.0, 1590.0, "fallback"
    try:
        with open(path) as f:
            d = json.load(f)
        hbm = float(d.get("hbm_gbs", hbm))
        flops = float(d.get("bf16_tflops", flops))
        src = "measured"
    except (OSError, ValueError):
        pass
    return hbm, flops, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [x.strip() for x in line.split(",")]))

    def mark(self):
        """The timed region starts here: earlier samples do not count."""
        self.t0 = time.perf_counter()

    def stop(self):
        if self.proc:
            time.sleep(0.05)
            self.proc.terminate()
        t0 = getattr(self, "t0", 0.0)
        self.rows = [r for t, r in self.rows if t >= t0] or [r for t, r in self.rows[-3:]]
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def model_numbers(cfg):
    """Matrix parameters read once per decode step, their flops per token, KV bytes per token."""
    H, F, V = cfg.hidden_size, cfg.ff_dim, cfg.vocab_size
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    n_attn = len(cfg.attention_layers)
    n_conv = cfg.num_hidden_layers - n_attn
    per_layer_ff = 3 * H * F
    conv = 3 * H * H + H * H
    attn = (Hq + 2 * Hkv) * D * H + Hq * D * H
    layer_params = cfg.num_hidden_layers * per_layer_ff + n_conv * conv + n_attn * attn
    head = V * H
    kv_bytes_per_token = n_attn * 2 * Hkv * D * 2
    state_bytes = n_conv * (cfg.conv_L_cache - 1) * H * 4
    return dict(layer_params=layer_params, head_params=head, kv_bytes_per_token=kv_bytes_per_token,
                state_bytes=state_bytes, n_attn=n_attn, attn_dims=(Hq, D))


PROFILE_RANGE = False      # --profile-range: the timed decode steps lie between cudaProfilerStart and cudaProfilerStop


def decode_requests(eng, B, steps_needed, seed):
    """Add B requests with contexts spread over CONTEXT / 2..CONTEXT and run until all of them decode."""
    from zig_ai_b200.sampling import SamplingParams
    g = random.Random(seed)
    lo = CONTEXT // 2
    hi = CONTEXT - steps_needed - 160          # room for the tokens decoded while later requests still prefill
    lens = [lo + (hi - lo) * i // max(B - 1, 1) for i in range(B)] if B > 1 else [(lo + hi) // 2]
    V = eng.config.vocab_size
    ids = [eng.add_request([g.randrange(V) for _ in range(n)],
                           SamplingParams(temperature=0.0, max_new_tokens=CONTEXT - n)) for n in lens]
    while any(eng.requests[i].computed < len(eng.requests[i].prompt) or not eng.requests[i].output for i in ids):
        eng.step()
    return ids


def time_decode(eng, B, steps, warmup, clocks=None):
    """Device-timed decode steps of batch B (step function + sampling kernel, no host read-back),
    then the same number of steps through Engine.step().  Returns (ms/step device, ms/step e2e,
    context tokens read per step, launches per step, h2d bytes, d2h bytes)."""
    import torch
    from zig_ai_b200.kernels import ops
    if clocks:
        clocks.start()                       # nvidia-smi takes a while to give its first sample
    ids = decode_requests(eng, B, 2 * (steps + warmup) + 4, seed=B)
    eng.flush()                              # no step on its way while the runner is driven directly
    reqs = [eng.requests[i] for i in ids]
    runner = eng.runner
    ctx_tokens = sum(r.computed for r in reqs)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    # the host work of every step (page reservation, packing) is done before the clock starts; the
    # timed region holds, per step, the pinned-to-device copy of the batch description, the step's
    # kernels and the sampling kernel, with no read-back in between
    prepared = [runner.prepare_decode([(r.request_id, [(7 * k + j) % 1000], [0]) for j, r in enumerate(reqs)])
                for k in range(warmup + steps)]
    for k in range(warmup):
        ops.argmax(runner.run_prepared(prepared[k]))
    torch.cuda.synchronize()
    launches0 = ops.launches
    if clocks:
        clocks.mark()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps - 1)]
    if PROFILE_RANGE:
        torch.cuda.profiler.start()          # a profiler started with --profile-from-start off sees only these steps
    start.record()
    for k in range(steps):
        ops.argmax(runner.run_prepared(prepared[warmup + k]))
        if k < steps - 1:
            marks[k].record()
    stop.record()
    torch.cuda.synchronize()
    if PROFILE_RANGE:
        torch.cuda.profiler.stop()
    dev_ms = start.elapsed_time(stop) / steps
    edges = [start] + marks + [stop]
    per_step = [edges[k].elapsed_time(edges[k + 1]) for k in range(steps)]
    launches = (ops.launches - launches0) / steps
    # the scheduler's view has to follow what was run behind its back
    for r in reqs:
        r.computed = runner.processed[r.request_id]
        r.output += [0] * (r.computed + 1 - len(r.prompt) - len(r.output))
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e2e_steps = []
    for _ in range(steps):
        t1 = time.perf_counter()
        eng.step()
        e2e_steps.append((time.perf_counter() - t1) * 1e3)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    if os.environ.get("ZAI_BENCH_STEPS"):
        worst = max(range(steps), key=lambda k: per_step[k])
        worst_e = max(range(steps), key=lambda k: e2e_steps[k])
        print(f"[bench] batch {B}: device median {sorted(per_step)[steps // 2]:.3f} ms, worst {per_step[worst]:.3f} ms at step "
              f"{worst}; e2e median {sorted(e2e_steps)[steps // 2]:.3f} ms, worst {e2e_steps[worst_e]:.3f} ms at step {worst_e}; "
              f"kernel status {ops.tc_status()}",
              file=sys.stderr, flush=True)
    clock_info = clocks.stop() if clocks else None
    eng.flush()
    for r in list(reqs):
        if r.request_id in eng.requests:
            eng.scheduler.running.remove(r)
            runner.end_request(r.request_id)
            eng.requests.pop(r.request_id)
    width = next(iter(runner.graphs.widths.values())) if runner.graphs else 0
    bucket = runner.graphs.bucket(B) if runner.graphs else B
    h2d = 4 * (3 * bucket + (bucket + 1) + 3 * bucket + bucket * width)
    d2h = 4 * (B + 1)                        # the token ids and the kernels' status word behind them
    return dev_ms, e2e_ms, ctx_tokens, launches, h2d, d2h, clock_info


def time_prefill(eng, reps=5):
    import torch
    g = random.Random(99)
    V = eng.config.vocab_size
    runner = eng.runner
    times = []
    for i in range(reps + 2):
        toks = [g.randrange(V) for _ in range(PREFILL_TOKENS)]
        rid = f"prefill{i}"
        runner.add_request(rid)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([(rid, toks, [PREFILL_TOKENS - 1])])
        stop.record()
        torch.cuda.synchronize()
        runner.end_request(rid)
        if i >= 2:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def run_ours(args):
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    from zig_ai_b200.kernels import build
    build.build_all(verbose=False)
    hbm_peak, flops_peak, peak_src = peaks()
    cfg = config_from_dict(shape_config(args.model))
    nums = model_numbers(cfg)
    if args.workload == "mixed":
        return run_mixed(args, cfg)
    if args.only == "long":
        return run_long(args)
    if args.only == "sample":
        return run_sample(args)
    if args.only == "table":
        return run_table(args)
    if args.only == "stream":
        return run_stream_table(cfg, args.batch)
    with tempfile.TemporaryDirectory(prefix="lfm2_350m_") as d:
        z.write_random_model(cfg, 0, d)
        eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048 + 64, max_model_len=CONTEXT,
                       max_tokens=64 * CONTEXT, page_size=args.page_size)
        if args.only == "gemm":
            return run_gemm_table(cfg)
        if args.only == "prefill":
            print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "ms": round(time_prefill(eng, reps=args.steps), 3)}))
            return 0
        if args.only == "timeline":
            return run_timeline(eng, args.batch)
        if args.only == "decode":
            ms, e2e, ctx, launches, _, _, _ = time_decode(eng, args.batch, args.steps, args.warmup)
            print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": round(ms, 4),
                              "e2e_ms_per_step": round(e2e, 4), "launches_per_step": launches}))
            return 0
        prefill_ms = time_prefill(eng, reps=15)
        clocks = ClockSampler()
        dev_ms, e2e_ms, ctx_tokens, launches, h2d, d2h, clock_info = time_decode(eng, 8, args.steps, args.warmup, clocks)
        points = {}
        for B in (1, 64):
            ms, _, _, _, _, _, _ = time_decode(eng, B, max(args.steps // 2, 20), args.warmup)
            points[f"decode_b{B}"] = round(B / ms * 1e3, 1)
    weight_bytes = 2 * (nums["layer_params"] + nums["head_params"])
    step_bytes = weight_bytes + ctx_tokens * nums["kv_bytes_per_token"] + 8 * nums["state_bytes"]
    achieved = step_bytes / (dev_ms * 1e-3) / 1e9
    Hq, D = nums["attn_dims"]
    T = PREFILL_TOKENS
    prefill_flops = 2 * T * nums["layer_params"] + 2 * 1 * nums["head_params"] + nums["n_attn"] * 2 * T * T * Hq * D
    out = {
        "metric": f"decode tok/s @ batch 8 (LFM2-{args.model.upper()} shape, context 2048-4096)",
        "value": round(8 / dev_ms * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)",
        "impl": "ours",
        "config": {"model": f"LFM2-{args.model.upper()} shape", "layers": cfg.num_hidden_layers, "layers_of_config": 16,
                   "attn_layers": nums["n_attn"], "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "ff_dim": cfg.ff_dim,
                   "vocab": cfg.vocab_size, "conv_taps": cfg.conv_L_cache, "global_batch": 8, "seq_len": CONTEXT,
                   "mean_context": round(ctx_tokens / 8), "page_size": args.page_size, "parallelism": "single GPU",
                   "l2": f"step reads {weight_bytes / 1e9:.2f} GB of weights (> 126 MB L2)", "peaks": peak_src},
        "e2e": {"value": round(8 / e2e_ms * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(round(launches * args.steps)),
        "prefill": {"value": round(T / prefill_ms * 1e3, 1), "tokens": T, "ms": round(prefill_ms, 3),
                    "frac": round(prefill_flops / (prefill_ms * 1e-3) / (flops_peak * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4)},
        "points": points,
        "clocks": clock_info,
    }
    print(json.dumps(out))
    return 0


def measure_shape(model, steps, warmup, page_size=64):
    """Every figure of one model shape: decode at batch 1, 8 and 64 (device-timed and through Engine.step),
    the prefill of 2048 tokens, each with the bytes or flops it has to move and the fraction of the peak."""
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    hbm_peak, flops_peak, peak_src = peaks()
    cfg = config_from_dict(shape_config(model))
    nums = model_numbers(cfg)
    rows = []
    with tempfile.TemporaryDirectory(prefix=f"lfm2_{model.replace('.', '_')}_") as d:
        z.write_random_model(cfg, 0, d)
        eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048 + 64, max_model_len=CONTEXT,
                       max_tokens=64 * CONTEXT, page_size=page_size)
        prefill_ms = time_prefill(eng, reps=max(min(steps, 20), 5))
        Hq, D = nums["attn_dims"]
        T = PREFILL_TOKENS
        flops = 2 * T * nums["layer_params"] + 2 * nums["head_params"] + nums["n_attn"] * 2 * T * T * Hq * D
        rows.append({"model": model, "point": "prefill 2048", "ms": round(prefill_ms, 3), "tokens_per_s": round(T / prefill_ms * 1e3),
                     "work": f"{flops / 1e12:.3f} TFLOP", "achieved": f"{flops / prefill_ms / 1e9:.0f} TFLOP/s",
                     "frac_of_peak": round(flops / (prefill_ms * 1e-3) / (flops_peak * 1e12), 3)})
        weight_bytes = 2 * (nums["layer_params"] + nums["head_params"])
        for B in (1, 8, 64):
            dev_ms, e2e_ms, ctx_tokens, launches, _, _, _ = time_decode(eng, B, max(steps, 20), warmup)
            step_bytes = weight_bytes + ctx_tokens * nums["kv_bytes_per_token"] + B * nums["state_bytes"]
            rows.append({"model": model, "point": f"decode batch {B}", "ms": round(dev_ms, 4), "e2e_ms": round(e2e_ms, 4),
                         "tokens_per_s": round(B / dev_ms * 1e3), "e2e_tokens_per_s": round(B / e2e_ms * 1e3),
                         "mean_context": round(ctx_tokens / B), "work": f"{step_bytes / 1e9:.3f} GB",
                         "achieved": f"{step_bytes / dev_ms / 1e6:.0f} GB/s",
                         "frac_of_peak": round(step_bytes / (dev_ms * 1e-3) / 1e9 / hbm_peak, 3),
                         "launches_per_step": round(launches)})
    return rows, peak_src


def run_table(args):
    """The tracked table: the 350M, 700M and 1.2B shapes, decode at batch 1/8/64 device-timed and end to end,
    the prefill of 2048 tokens, and the mixed workload of the 700M shape, as JSON lines and as markdown."""
    hbm_peak, flops_peak, peak_src = peaks()
    all_rows = []
    for model in ("350m", "700m", "1.2b"):
        rows, _ = measure_shape(model, args.steps, args.warmup, args.page_size)
        for r in rows:
            print(json.dumps(r), flush=True)
        all_rows += rows
    print(f"\npeaks ({peak_src}): {hbm_peak:.0f} GB/s copy bandwidth, {flops_peak:.0f} TFLOP/s bf16 product (burst)\n")
    print("| shape | point | ms a step (device) | tokens/s (device) | ms a step (end to end) | tokens/s (end to end) | bytes or flops a step | achieved | of the measured peak |")
    print("|---|---|---|---|---|---|---|---|---|")
    for r in all_rows:
        print(f"| LFM2-{r['model'].upper()} | {r['point']} | {r['ms']} | {r['tokens_per_s']} | {r.get('e2e_ms', '')} | "
              f"{r.get('e2e_tokens_per_s', '')} | {r['work']} | {r['achieved']} | {r['frac_of_peak']} |")
    return 0


def run_long(args):
    """Further context lengths (one shape, --model): a prompt of --context tokens prefilled in portions of 2048
    (each portion timed: its products are the same, its attention grows with the cached context), and decode
    steps at batch 8 with contexts spread over the upper half of --context."""
    global CONTEXT
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    hbm_peak, flops_peak, peak_src = peaks()
    cfg = config_from_dict(shape_config(args.model))
    nums = model_numbers(cfg)
    CONTEXT = args.context
    B = 8
    with tempfile.TemporaryDirectory(prefix="lfm2_long_") as d:
        z.write_random_model(cfg, 0, d)
        eng = z.Engine(d, "bfloat16", max_num_seqs=B, max_batched_tokens=2048 + 64, max_model_len=CONTEXT,
                       max_tokens=(B + 1) * CONTEXT, page_size=args.page_size)
        runner = eng.runner
        g = random.Random(5)
        Hq, D = nums["attn_dims"]
        T = PREFILL_TOKENS
        for rep in range(2):                                   # the first pass warms up (graphs of the portions' shapes are captured)
            rid = f"long{rep}"
            runner.add_request(rid)
            portions = []
            for c in range(CONTEXT // T):
                toks = [g.randrange(cfg.vocab_size) for _ in range(T)]
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                start.record()
                runner.step([(rid, toks, [T - 1])])
                stop.record()
                torch.cuda.synchronize()
                portions.append(start.elapsed_time(stop))
            runner.end_request(rid)
        total_ms = sum(portions)
        # flops: every portion's products, and attention of its 2048 rows over the cached context and itself
        products = 2 * T * nums["layer_params"] + 2 * nums["head_params"]
        attn = [nums["n_attn"] * 2 * 2 * Hq * D * (T * c * T + T * T // 2) for c in range(CONTEXT // T)]
        flops = len(portions) * products + sum(attn)
        print(json.dumps({"only": "long", "model": args.model, "point": f"prefill {CONTEXT} in portions of {T}",
                          "ms": round(total_ms, 2), "tokens_per_s": round(CONTEXT / total_ms * 1e3),
                          "first_portion_ms": round(portions[0], 3), "last_portion_ms": round(portions[-1], 3),
                          "tflop": round(flops / 1e12, 2), "achieved_tflops": round(flops / total_ms / 1e9),
                          "frac_of_peak": round(flops / (total_ms * 1e-3) / (flops_peak * 1e12), 3),
                          "last_portion_attention_share_of_flops": round(attn[-1] / (products + attn[-1]), 3),
                          "last_portion_frac_of_peak": round((products + attn[-1]) / (portions[-1] * 1e-3) / (flops_peak * 1e12), 3),
                          "peaks": peak_src}), flush=True)
        weight_bytes = 2 * (nums["layer_params"] + nums["head_params"])
        dev_ms, e2e_ms, ctx_tokens, launches, _, _, _ = time_decode(eng, B, max(args.steps, 20), args.warmup)
        step_bytes = weight_bytes + ctx_tokens * nums["kv_bytes_per_token"] + B * nums["state_bytes"]
        print(json.dumps({"only": "long", "model": args.model, "point": f"decode batch {B}", "mean_context": round(ctx_tokens / B),
                          "ms": round(dev_ms, 4), "e2e_ms": round(e2e_ms, 4), "tokens_per_s": round(B / dev_ms * 1e3),
                          "e2e_tokens_per_s": round(B / e2e_ms * 1e3), "gb": round(step_bytes / 1e9, 3),
                          "achieved_gbs": round(step_bytes / dev_ms / 1e6),
                          "frac_of_peak": round(step_bytes / (dev_ms * 1e-3) / 1e9 / hbm_peak, 3), "peaks": peak_src}), flush=True)
    return 0


def run_sample(args):
    """Sampling: the kernel alone at the shape's vocabulary (1, 8 and 64 rows; twenty eager calls, so about 13 us
    of each figure are the launch), and decode steps through Engine.step() with sampled requests."""
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.config import config_from_dict
    from zig_ai_b200.kernels import ops
    from zig_ai_b200.sampling import SamplingParams
    cfg = config_from_dict(shape_config(args.model))
    V = cfg.vocab_size
    ops.require(torch.bfloat16)
    kinds = (("temperature 0.8", 0, 1.0), ("top-k 40", 40, 1.0), ("top-p 0.9", 0, 0.9), ("top-k 40, top-p 0.9", 40, 0.9))
    for R in (1, 8, 64):
        logits = torch.randn(R, V, device="cuda") * 3
        row = {"only": "sample", "rows": R, "vocab": V}
        for name, tk, tp in kinds:
            t = torch.full((R,), 0.8, device="cuda")
            k = torch.full((R,), tk, dtype=torch.int32, device="cuda")
            p = torch.full((R,), tp, device="cuda")
            u = torch.rand(R, device="cuda")
            for _ in range(3):
                ops.sample(logits, t, k, p, u)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(20):
                ops.sample(logits, t, k, p, u)
            b.record()
            torch.cuda.synchronize()
            row[name + " us"] = round(a.elapsed_time(b) * 50, 1)
        print(json.dumps(row), flush=True)
    g = random.Random(3)
    with tempfile.TemporaryDirectory(prefix="lfm2_sample_") as d:
        z.write_random_model(cfg, 0, d)
        for name, sp in (("greedy", dict(temperature=0.0)), ("temperature 0.8", dict(temperature=0.8)),
                         ("temperature 0.8, top-k 40, top-p 0.9", dict(temperature=0.8, top_k=40, top_p=0.9)),
                         ("and repetition penalty 1.1", dict(temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.1))):
            eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048 + 64, max_model_len=CONTEXT, max_tokens=64 * CONTEXT)
            row = {"only": "sample", "requests": name}
            for B in (8, 64):
                ids = [eng.add_request([g.randrange(V) for _ in range(2048 + 20 * i)], SamplingParams(max_new_tokens=300, seed=i, **sp))
                       for i in range(B)]
                while any(eng.requests[i].computed < len(eng.requests[i].prompt) or not eng.requests[i].output for i in ids):
                    eng.step()
                for _ in range(20):
                    eng.step()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(100):
                    eng.step()
                torch.cuda.synchronize()
                row[f"ms a step at batch {B}"] = round((time.perf_counter() - t0) * 10, 4)
                while eng.has_work():
                    eng.step()
            print(json.dumps(row), flush=True)
            del eng
    return 0


def run_timeline(eng, B):
    """One decode step's kernels on the device's own clock (libraries built with ZAI_TIMELINE=1): when
    each kernel's first block was resident and waiting, when its wait for the kernel before it ended,
    and how long until the next kernel's wait ended (its share of the step)."""
    import collections
    from zig_ai_b200.kernels import ops
    ids = decode_requests(eng, B, 40, seed=B)
    eng.flush()
    reqs = [eng.requests[i] for i in ids]
    runner = eng.runner
    prepared = [runner.prepare_decode([(r.request_id, [(7 * k + j) % 1000], [0]) for j, r in enumerate(reqs)])
                for k in range(12)]
    for k in range(10):
        ops.argmax(runner.run_prepared(prepared[k]))
    ops.timeline()
    for k in range(10, 12):
        ops.argmax(runner.run_prepared(prepared[k]))
    tl = [r for r in ops.timeline() if " mark " not in r[0] and " block " not in r[0]]
    starts = [i for i, r in enumerate(tl) if r[0] == "embed_kernel"]
    step = tl[starts[-1]:]
    t0 = step[0][2]
    print(f"batch {B}: {len(step)} kernels, {(step[-1][2] - t0) / 1e3:.1f} us from the first kernel's start to the last one's")
    print("  # kernel                                   resident at   wait over   waited   until next (us)")
    agg = collections.OrderedDict()
    for i, (name, a, b) in enumerate(step):
        nxt = step[i + 1][2] if i + 1 < len(step) else b
        print(f"{i:3d} {name:40s} {(a - t0) / 1e3:10.2f} {(b - t0) / 1e3:11.2f} {(b - a) / 1e3:8.2f} {(nxt - b) / 1e3:8.2f}")
        e = agg.setdefault(name, [0, 0.0])
        e[0] += 1
        e[1] += (nxt - b) / 1e3
    print("by kernel (launches, us in the step, us each):")
    for name, (n, us) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        print(f"  {name:40s} {n:3d} {us:8.1f} {us / n:7.2f}")
    return 0


def run_gemm_table(cfg):
    """The products of the model's layers at 2048, 512 and 128 rows: the tcgen05 kernel of this package
    against the library's product (plus the activation kernel where the tcgen05 kernel fuses it), each
    timed as a CUDA graph of 20 calls that rotate over copies of the weights (so they come from HBM)."""
    import ctypes
    import torch
    from zig_ai_b200.kernels import ops
    ops.require()
    fn = ops._fn("gemm_tc", "zai_gemm_tc")
    fn2 = ops._fn("gemm_tc_pair", "zai_gemm_pair")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    H, F = cfg.hidden_size, cfg.ff_dim
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    shapes = [("out_proj", H, H, 0), ("qkv", qkv, H, 0), ("in_proj", 3 * H, H, 0), ("gate_up+swiglu", 2 * F, H, 2), ("down", H, F, 0)]

    def graph_time(f, reps=20):
        for _ in range(2):
            f()
        torch.cuda.synchronize()
        g, s = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(s):
            with torch.cuda.graph(g):
                ops.begin_forward()
                for _ in range(reps):
                    f()
                ops.end_forward()
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (5 * reps) * 1e3

    rows = []
    for N in (2048, 512, 128):
        for name, O, K, epi in shapes:
            ws = [torch.randn(O, K).to(torch.bfloat16).cuda() for _ in range(max(2, min(8, int(200e6 // (O * K * 2)))))]
            x = torch.randn(N, K).to(torch.bfloat16).cuda()
            y = torch.empty((N, O // 2 if epi == 2 else O), dtype=torch.bfloat16, device="cuda")
            it = [0]

            def tc():
                w = ws[it[0] % len(ws)]
                it[0] += 1
                fn(y.data_ptr(), w.data_ptr(), x.data_ptr(), status.data_ptr(), N, O, K, epi, ops._stream())

            def lib():
                w = ws[it[0] % len(ws)]
                it[0] += 1
                if epi == 2:
                    ops.silu_mul(torch.matmul(x, w.t()), O // 2)
                else:
                    torch.matmul(x, w.t())
            def pair(wide):
                def f():
                    w = ws[it[0] % len(ws)]
                    it[0] += 1
                    fn2(y.data_ptr(), w.data_ptr(), x.data_ptr(), status.data_ptr(), N, O, K, epi, wide, ops._stream())
                return f
            t, t2 = graph_time(tc), graph_time(lib)
            tw, tn = graph_time(pair(1)), graph_time(pair(0))
            tp = min(tw, tn)
            rows.append({"rows": N, "product": name, "O": O, "K": K, "pair_us": round(tp, 1), "pair_wide_us": round(tw, 1),
                         "pair_narrow_us": round(tn, 1), "pair_tflops": round(2 * N * O * K / tp / 1e6),
                         "tcgen05_us": round(t, 1),
                         "tcgen05_tflops": round(2 * N * O * K / t / 1e6), "library_us": round(t2, 1),
                         "library_tflops": round(2 * N * O * K / t2 / 1e6)})
            print(json.dumps(rows[-1]))
    print(json.dumps({"only": "gemm", "status": int(status.item())}))
    return 0


def run_stream_table(cfg, only_rows=0):
    """The products of a layer at 24, 64 and 128 rows: the weight-streaming tcgen05 kernel of this package
    (csrc/stream_gemm.cu, with SwiGLU fused where the layer has it) against the library's product (plus the
    activation kernel), each timed as a CUDA graph of 20 calls that rotate over copies of the weights."""
    import torch
    from zig_ai_b200.kernels import ops
    ops.require()
    ops.USE_STREAM_GEMM = True
    H, F = cfg.hidden_size, cfg.ff_dim
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    shapes = [("out_proj", H, H, 0), ("qkv", qkv, H, 0), ("in_proj", 3 * H, H, 0), ("gate_up+swiglu", 2 * F, H, 2), ("down", H, F, 0),
              ("head", cfg.vocab_size, H, 1)]

    def graph_time(f, reps=20):
        for _ in range(2):
            f()
        torch.cuda.synchronize()
        g, s = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(s):
            with torch.cuda.graph(g):
                ops.begin_forward()
                for _ in range(reps):
                    f()
                ops.end_forward()
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (5 * reps) * 1e3

    for N in ((only_rows,) if only_rows in (24, 64, 128) else (24, 64, 128)):
        for name, O, K, epi in shapes:
            ws = [torch.randn(O, K).to(torch.bfloat16).cuda() for _ in range(max(2, min(8, int(300e6 // (O * K * 2)))))]
            x = torch.randn(N, K).to(torch.bfloat16).cuda()
            it = [0]

            def mine():
                w = ws[it[0] % len(ws)]
                it[0] += 1
                if epi == 2:
                    ops.linear_swiglu(x, w, O // 2)
                else:
                    ops.linear(x, w, torch.float32 if epi == 1 else None)

            def lib():
                w = ws[it[0] % len(ws)]
                it[0] += 1
                if epi == 2:
                    ops.silu_mul(torch.matmul(x, w.t()), O // 2)
                elif epi == 1:
                    torch.mm(x, w.t(), out_dtype=torch.float32)
                else:
                    torch.matmul(x, w.t())
            t1, t2 = graph_time(mine), graph_time(lib)
            print(json.dumps({"rows": N, "product": name, "O": O, "K": K, "stream_us": round(t1, 2), "library_us": round(t2, 2),
                              "stream_GBs": round(O * K * 2 / t1 / 1e3)}), flush=True)
    print(json.dumps({"only": "stream", "status": ops.read_status()}))
    return 0


def run_mixed(args, cfg):
    """64 requests with prompts of 256..2048 random tokens and 256 new tokens each, chunked prefill
    interleaved with decoding, through Engine.step(): tokens per second end to end."""
    import torch
    import zig_ai_b200 as z
    from zig_ai_b200.sampling import SamplingParams
    g = random.Random(7)
    with tempfile.TemporaryDirectory(prefix="lfm2_mixed_") as d:
        z.write_random_model(cfg, 0, d)
        eng = z.Engine(d, "bfloat16", max_num_seqs=64, max_batched_tokens=2048, max_model_len=CONTEXT,
                       max_tokens=64 * 2560)
        V = cfg.vocab_size
        for rep in range(2):                       # the first pass warms up graphs and allocator
            prompts = [[g.randrange(V) for _ in range(g.randint(256, 2048))] for _ in range(64)]
            ids = [eng.add_request(p, SamplingParams(temperature=0.0, max_new_tokens=256)) for p in prompts]
            torch.cuda.synchronize()
            t0, steps0, done = time.perf_counter(), eng.n_steps, 0
            while done < len(ids):
                done += len(eng.step())
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        n_prompt = sum(len(p) for p in prompts)
        st = eng.stats()
    out = {"metric": f"mixed workload tok/s (LFM2-{args.model.upper()} shape, 64 requests, prompts 256-2048, 256 new tokens each)",
           "value": round(64 * 256 / dt, 1), "unit": "generated tokens/s", "n_gpus": 1, "seconds": round(dt, 3),
           "prompt_tokens": n_prompt, "prompt_tokens_per_s": round(n_prompt / dt, 1), "steps": eng.n_steps - steps0,
           "mean_step_ms": round(dt * 1e3 / max(eng.n_steps - steps0, 1), 3),
           "pages_high_water": max(v for k, v in st.items() if k.endswith("pages_high_water")),
           "preemptions": st["preemptions"], "step_graph_replays": eng.runner.shape_graphs.replays,
           "step_graphs_kept": len(eng.runner.shape_graphs.graphs), "dtype": "bf16", "data": "synthetic", "impl": "ours"}
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "gemm", "timeline", "table", "stream", "long", "sample"],
                    help="profiling aid: run only the batch-8 decode steps or only the prefill (prints a short line); "
                         "table: every figure of the 350M, 700M and 1.2B shapes (profiles/measurements.md)")
    ap.add_argument("--batch", type=int, default=8, help="with --only decode: the batch size; with --only stream: 24, 64 or "
                                                         "128 runs that row count only")
    ap.add_argument("--profile-range", action="store_true",
                    help="mark the device-timed decode steps for a profiler (ncu --profile-from-start off)")
    ap.add_argument("--page-size", type=int, default=64, help="positions per cache page")
    ap.add_argument("--context", type=int, default=32768, help="with --only long: the context length (a multiple of 2048)")
    ap.add_argument("--model", default="350m", choices=sorted(SHAPES), help="which LFM2 shape (default: the 350M shape)")
    ap.add_argument("--workload", default="steps", choices=["steps", "mixed"],
                    help="mixed: 64 requests, chunked prefill interleaved with decoding, end to end")
    args = ap.parse_args()
    global PROFILE_RANGE
    PROFILE_RANGE = args.profile_range
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Zig 0.16 program (build.zig); no Zig compiler exists in this image and it "
                          "has no Python package to install, and it publishes no LFM2 figures"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    args.warmup = max(args.warmup, 3)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
