"""Trace replay over the engine's own step function (see bin/trace_run).

The reference has no such program; it dumps logits and per-layer activations by hand through
environment switches (`DUMP_LOGITS`, `DUMP_PREFILL_LAYERS`, src/main.zig:854-860, 1336-1338).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids through the engine and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--max-requests", type=int, default=8)
    ap.add_argument("--stats", default=None, metavar="FILE",
                    help="when the input ends, write the cache's and the runner's counters to FILE as JSON")
    args = ap.parse_args(argv)

    from .runner import load_runner
    os.makedirs(args.out, exist_ok=True)
    runner = load_runner(args.model, args.dtype, max_tokens=args.max_tokens, max_requests=args.max_requests,
                         page_size=args.page_size)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            if not runner.has_request(e["id"]):
                runner.add_request(e["id"])
            entries.append((e["id"], e["tokens"], e.get("want", [])))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                data = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
                with open(os.path.join(args.out, f"{step}.f32"), "wb") as f:
                    f.write(data.tobytes())
            else:
                torch.cuda.synchronize()
        for rid in rec.get("end", []):
            if runner.has_request(rid):
                runner.end_request(rid)
        print(f"done {step}", flush=True)
    if args.stats:
        stats = dict(runner.cache.stats(), steps=runner.steps, tokens_run=runner.tokens_run,
                     num_pages=runner.cache.num_pages, page_size=runner.cache.page_size)
        with open(args.stats, "w") as f:
            json.dump(stats, f)
    return 0
