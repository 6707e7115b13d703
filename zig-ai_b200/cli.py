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
    eng = Engine(args.model, args.dtype, max_num_seqs=max(len(prompts), 1),
                 max_batched_tokens=min(args.batch_size, max(args.ubatch_size, 1) + len(prompts)),
                 max_model_len=args.max_model_len or longest)
    print(f"[+] model {args.model}: {eng.config.architecture}, dtype {args.dtype}, {len(prompts)} sequence(s)")
    ids = [eng.add_request(p, SamplingParams(
        temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
        repetition_penalty=args.repetition_penalty, seed=args.seed + i, max_new_tokens=args.max_tokens,
        eos_id=args.eos_id)) for i, p in enumerate(prompts)]
    done, t0, t_first = {}, time.perf_counter(), None
    while len(done) < len(ids):
        for r in eng.step():
            done[r.request_id] = r
        if t_first is None and eng.n_generated > 0:
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
    print(f"[+] prefill: {n_prompt} tokens in {prefill_ms:.1f} ms ({n_prompt / max(prefill_ms, 1e-6) * 1e3:.1f} tok/s)")
    print(f"[+] decode: {max(n_gen - len(ids), 0)} tokens in {decode_s * 1e3:.1f} ms "
          f"({max(n_gen - len(ids), 0) / decode_s:.1f} tok/s)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
