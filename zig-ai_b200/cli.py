"""Command line in the manner of the reference's `zig-ai-engine` (src/main.zig:177-319): the same
names and meanings for the options it shares with this engine.

    -m, --model DIR            model folder (config.json, model.safetensors)
    --prompt IDS               prompt as token ids, "1,2,3" or "1 2 3" (the tokenizer is not part of this engine)
    -n, --max-tokens N         tokens to generate (default 128)
    --temperature F            default 1.0; <= 0 is greedy
    --top-k N                  default 0 (off)
    --top-p F                  default 1.0 (off)
    --repetition-penalty F     default 1.0 (off)
    --seed N                   default 42
    --backend auto|gpu|cpu     auto and gpu run on the B200; cpu is refused (there is no CPU path)
    -np N                      parallel sequences of the same prompt, seeds seed..seed+N-1 (default 1)
    -b, --batch-size N         tokens per step (default 2048)
    -ub, --ubatch-size N       largest prompt portion per step (default 512)
    --page-size N              positions per cache page (default 64; the reference's BLOCK_SIZE = 16, src/main.zig:604)
    --num-pages N              pages of the pool (default: room for every sequence at --max-model-len;
                               the reference's MAX_BLOCKS_GPU, src/main.zig:605-611)
    --max-num-seqs N           sequences that run at once (default: as many as there are prompts)
    --profile                  time every step's kernels by class and print the table (PERF_STAGE, src/main.zig:817-931)
    --allow-unused-tensors     stored tensors that the model does not ask for are passed over with a note

Options of the reference that belong to features outside this engine (-ctk/-ctv, --spec-*, --quant,
--layer-stream*, -ngl, -jinja) are accepted and ignored with a note.
"""
from __future__ import annotations

import argparse
import re
import sys
import time


def parse_ids(text: str):
    parts = [p for p in re.split(r"[,\s]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit("--prompt takes token ids (\"1,2,3\"); text prompts need a tokenizer, which this engine leaves out")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="zig-ai-engine", description="LFM2 inference on one B200")
    ap.add_argument("-m", "--model", help="model folder (config.json, model.safetensors)")
    ap.add_argument("--prompt", default=None, help="token ids, e.g. \"1,2,3\"")
    ap.add_argument("--prompt-file", default=None, help="file with one prompt (token ids) per line")
    ap.add_argument("-n", "--max-tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--backend", default="auto", choices=["auto", "cpu", "gpu"])
    ap.add_argument("-np", type=int, default=1, dest="num_parallel")
    ap.add_argument("-b", "--batch-size", type=int, default=2048)
    ap.add_argument("-ub", "--ubatch-size", type=int, default=512)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-model-len", type=int, default=None)
    ap.add_argument("--eos-id", type=int, default=None)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--num-pages", type=int, default=None)
    ap.add_argument("--max-num-seqs", type=int, default=None)
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--allow-unused-tensors", action="store_true")
    ap.add_argument("--random-weights", metavar="CONFIG_JSON", default=None,
                    help="write a model folder with random weights for this config.json into --model and use it")
    for flag in ("-ctk", "--cache-type-k", "-ctv", "--cache-type-v", "--spec-draft-type-k", "--spec-draft-type-v",
                 "--spec-type", "--spec-draft-n-max", "--quant", "--layer-stream-max", "-ngl", "--n-gpu-layers",
                 "--gpu-layers"):
        ap.add_argument(flag, dest="ignored_" + flag.strip("-").replace("-", "_"), default=None)
    for flag in ("--layer-stream", "-jinja", "--jinja"):
        ap.add_argument(flag, dest="ignored_" + flag.strip("-").replace("-", "_"), action="store_true")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    for k, v in vars(args).items():
        if k.startswith("ignored_") and v:
            print(f"[!] option {k[8:].replace('_', '-')} belongs to a feature this engine leaves out; ignored")
    if args.backend == "cpu":
        print("[!] this engine has no CPU path; use --backend auto or gpu")
        return 2
    if not args.model:
        build_parser().print_help()
        return 0
    if args.random_weights:
        from .config import load_config
        from .weights import write_random_model
        write_random_model(load_config(args.random_weights), args.seed, args.model)
        print(f"[+] wrote random weights (seed {args.seed}) to {args.model}")
    prompts = []
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts = [parse_ids(line) for line in f if line.strip()]
    elif args.prompt is not None:
        prompts = [parse_ids(args.prompt)]
    else:
        prompts = [[0]]
    prompts = [p for p in prompts for _ in range(max(args.num_parallel, 1))]

    from .engine.engine import Engine
    from .sampling.sampler import SamplingParams
    import torch
    longest = max(len(p) for p in prompts) + args.max_tokens
    if args.page_size < 1 or (args.num_pages is not None and args.num_pages < 1) or \
            (args.max_num_seqs is not None and args.max_num_seqs < 1):
        print("[!] --page-size, --num-pages and --max-num-seqs take positive numbers")
        return 2
    n_seqs = args.max_num_seqs or max(len(prompts), 1)
    eng = Engine(args.model, args.dtype, max_num_seqs=n_seqs,
                 max_batched_tokens=min(args.batch_size, max(args.ubatch_size, 1) + n_seqs),
                 max_model_len=args.max_model_len or longest, page_size=args.page_size,
                 max_tokens=args.num_pages * args.page_size if args.num_pages else None, profile=args.profile,
                 unexpected_tensors="warn" if args.allow_unused_tensors else "error")
    print(f"[+] model {args.model}: {eng.config.architecture}, dtype {args.dtype}, {len(prompts)} sequence(s)")
    if torch.cuda.is_available() and not args.profile:
        t_w = time.perf_counter()
        eng.warm_up(min(len(prompts), n_seqs))               # (first calls and the decode graph: not the prompts' time)
        torch.cuda.synchronize()
        print(f"[+] warm-up: {(time.perf_counter() - t_w) * 1e3:.0f} ms")
    ids = [eng.add_request(p, SamplingParams(
        temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
        repetition_penalty=args.repetition_penalty, seed=args.seed + i, max_new_tokens=args.max_tokens,
        eos_id=args.eos_id)) for i, p in enumerate(prompts)]
    gen0 = eng.n_generated
    done, t0, t_first = {}, time.perf_counter(), None
    while len(done) < len(ids):
        for r in eng.step():
            done[r.request_id] = r
        if t_first is None and eng.n_generated > gen0:
            torch.cuda.synchronize()
            t_first = time.perf_counter()
    eng.flush()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    for i in ids:
        print(f"[{i}] ({done[i].finish_reason}) " + " ".join(str(t) for t in done[i].output))
    n_gen = sum(len(done[i].output) for i in ids)
    n_prompt = sum(len(p) for p in prompts)
    prefill_ms = ((t_first or t1) - t0) * 1e3
    decode_s = max(t1 - (t_first or t1), 1e-9)
    if len(ids) == 1:
        print(f"[+] prefill: {n_prompt} tokens in {prefill_ms:.1f} ms ({n_prompt / max(prefill_ms, 1e-6) * 1e3:.1f} tok/s)")
        print(f"[+] decode: {max(n_gen - len(ids), 0)} tokens in {decode_s * 1e3:.1f} ms "
              f"({max(n_gen - len(ids), 0) / decode_s:.1f} tok/s)")
    else:
        # with several prompts their portions run beside the decoding of the ones that are through, so there is no
        # prefill time apart from the decode time: the first token's time, and the whole
        total_s = max(t1 - t0, 1e-9)
        print(f"[+] prefill: first token after {prefill_ms:.1f} ms; {n_prompt} prompt tokens in portions beside decoding")
        print(f"[+] decode: {n_gen} tokens of {len(ids)} sequences in {total_s * 1e3:.1f} ms ({n_gen / total_s:.1f} tok/s; "
              f"{(n_gen + n_prompt) / total_s:.1f} tok/s with the prompts)")
    st = eng.stats()
    print(f"[+] cache: {eng.runner.cache.num_pages} pages of {args.page_size} positions, high water "
          + ", ".join(f"{v}" for k, v in st.items() if k.endswith("_pages_high_water")) + f"; {st['preemptions']} preemption(s)")
    if args.profile:
        print_profile(eng.profile_report())
    return 0


def print_profile(report) -> None:
    """Per kind of step: milliseconds a step by kernel class (steps launched kernel by kernel)."""
    for kind, acc in report.items():
        steps = max(int(acc.get("steps", 0)), 1)
        rows = sorted(((k, v) for k, v in acc.items() if k not in ("steps", "tokens")), key=lambda kv: -kv[1])
        total = sum(v for _, v in rows)
        print(f"[profile] {kind}: {steps} step(s), {int(acc.get('tokens', 0))} tokens, {total / steps:.3f} ms of kernels a step")
        for k, v in rows:
            print(f"[profile]   {k:<48s} {v / steps:9.3f} ms  {100 * v / max(total, 1e-12):5.1f} %")


if __name__ == "__main__":
    sys.exit(main())
