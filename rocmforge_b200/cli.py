"""Command line in the manner of maeddesg/ROCmForge's one-shot binary (src/main.rs:42-144).

Flags it has keep their names, meanings and defaults: --model/-m, --prompt/-p,
--max-tokens (256), --temperature/-t/--temp (1.0), --top-p (0.9), --no-template,
--list-tensors, --debug, --gpu.  --model names a folder with config.json and safetensors
instead of a GGUF file; --gpu and --no-template are accepted and change nothing (this engine
has only a GPU path and no chat templates).  Greedy decoding is selected by
--temperature 0, the rule of the reference's chat loop (src/cli/chat.rs:483).
Added: --prompt-ids, --top-k, --seed, --dtype, --stop-ids, --random-config/--random-seed.
Text goes through a byte-level stand-in tokenizer.  The two statistics lines on stderr
are the reference's (src/main.rs:729-734, :989-994).
"""
from __future__ import annotations

import argparse
import sys
import time


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="rocmforge", description="B200-native generation for Qwen2.5 models")
    ap.add_argument("-m", "--model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("-p", "--prompt", action="append", default=[], help="input prompt (repeat for a batch)")
    ap.add_argument("--prompt-ids", action="append", default=[], help="prompt as comma-separated token ids")
    ap.add_argument("--max-tokens", type=int, default=256, help="maximum tokens to generate [default: 256]")
    ap.add_argument("-t", "--temp", "--temperature", dest="temperature", type=float, default=1.0,
                    help="sampling temperature, 0 = greedy [default: 1.0]")
    ap.add_argument("--top-p", type=float, default=0.9, help="nucleus sampling threshold [default: 0.9]")
    ap.add_argument("--top-k", type=int, default=0, help="keep the k most likely tokens, 0 = off")
    ap.add_argument("--seed", type=lambda s: int(s, 0), default=0xDEADBEEF, help="sampler seed")
    ap.add_argument("--no-template", action="store_true", help="accepted; prompts are always raw")
    ap.add_argument("--list-tensors", action="store_true", help="list tensors in the model folder and exit")
    ap.add_argument("--debug", action="store_true", help="show the generated token ids as they come")
    ap.add_argument("--gpu", action="store_true", help="accepted; this engine always runs on the GPU")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--stop-ids", default=None, help="comma-separated stop token ids (default: eos_token_id)")
    ap.add_argument("--random-config", help="config.json of a model to fill with random weights")
    ap.add_argument("--random-seed", type=int, default=0)
    ap.add_argument("--write-random", metavar="DIR",
                    help="with --random-config: write config.json and model.safetensors to DIR and exit")
    return ap


def list_tensors(folder: str) -> int:
    # src/main.rs:148-162 — name, dtype, shape of every tensor
    from .weights import ModelFiles
    files = ModelFiles(folder)
    for name in sorted(files.names()):
        e = files.entries[name]
        print(f"{name}\t{str(e.dtype).replace('torch.', '')}\t{list(e.shape)}")
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.list_tensors:
        if not args.model:
            print("--list-tensors needs --model", file=sys.stderr)
            return 1
        return list_tensors(args.model)

    import torch
    from . import write_model_folder
    from .api import LLM, decode_bytes
    from .config import load_config

    if args.random_config and args.write_random:
        arch, cfg = load_config(args.random_config)
        dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
        write_model_folder(args.write_random, cfg.to_dict(), arch.build(cfg).param_specs(), args.random_seed, dt)
        print(f"wrote {args.write_random}", file=sys.stderr)
        return 0
    if not args.model and not args.random_config:
        print("Error: --model <folder> (or --random-config <config.json>) is required", file=sys.stderr)
        return 1
    if not args.prompt and not args.prompt_ids:
        print("Error: --prompt <text> or --prompt-ids <ids> is required", file=sys.stderr)
        return 1
    try:
        if args.model:
            llm = LLM(args.model, dtype=args.dtype)
        else:
            _, cfg = load_config(args.random_config)
            llm = LLM.random(cfg, args.random_seed, dtype=args.dtype)
        prompts = list(args.prompt) + [[int(t) for t in s.split(",") if t.strip()] for s in args.prompt_ids]
        stops = None if args.stop_ids is None else [int(t) for t in args.stop_ids.split(",") if t.strip()]
        first = {}
        t0 = time.perf_counter()

        def on_token(i, tok):
            if i not in first:
                first[i] = time.perf_counter() - t0
            if args.debug:
                print(f"[Generated] request={i} token_id={tok}", file=sys.stderr)

        results = llm.generate(prompts, max_tokens=args.max_tokens, temperature=args.temperature,
                               top_p=args.top_p, top_k=args.top_k, seed=args.seed, stop_token_ids=stops,
                               on_token=on_token)
    except Exception as e:                       # src/main.rs:1028-1064 — message and exit code 1
        print(f"Error: {e}", file=sys.stderr)
        return 1
    total = time.perf_counter() - t0
    for i, r in enumerate(results):
        head = f"[{i}] " if len(results) > 1 else ""
        print(head + decode_bytes(r.tokens))
    n_prompt = sum(r.prompt_len for r in results)
    n_gen = sum(len(r.tokens) for r in results)
    if first:
        ttft = max(first.values())
        print(f"Prefill: {ttft * 1e3:.1f}ms ({n_prompt / ttft:.1f} tok/s)", file=sys.stderr)
        gen = max(total - ttft, 1e-9)
        print(f"\n{n_gen} tokens in {gen * 1e3:.1f}ms = {n_gen / gen:.1f} tok/s", file=sys.stderr)
    for i, r in enumerate(results):
        print(f"[{i}] {len(r.tokens)} tokens, ended by {r.reason}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
