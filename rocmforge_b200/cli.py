"""Command line in the manner of maeddesg/ROCmForge's one-shot binary (src/main.rs:42-144).

Flags it has keep their names, meanings and defaults: --model/-m, --prompt/-p,
--max-tokens (256), --temperature/-t/--temp (1.0), --top-p (0.9), --no-template,
--list-tensors, --debug, --gpu.  --model names a folder with config.json and safetensors
instead of a GGUF file; --gpu and --no-template are accepted and change nothing (this engine
has only a GPU path and no chat templates).  Greedy decoding is selected by
--temperature 0, the rule of the reference's chat loop (src/cli/chat.rs:483).
--debug prints, as the reference does (src/main.rs:165-207, :725-727, :954-957), the most likely
tokens with their probabilities after the prompt (ten) and for the first steps (five each), or the
count of NaN and Inf logits with minimum, maximum and mean if there are any; the logits are then
looked at step by step, outside the replayed graphs.
Added: --prompt-ids, --prompt-len, --top-k, --seed, --dtype, --stop-ids, --no-graph, --stats-json,
--random-config/--random-seed.  Text goes through a byte-level stand-in tokenizer.  The two
statistics lines on stderr are the reference's (src/main.rs:729-734, :989-994).
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
    ap.add_argument("--debug", action="store_true",
                    help="show the most likely tokens (or the NaN/Inf count) of the prompt and the first steps, and every token id")
    ap.add_argument("--prompt-len", action="append", type=int, default=[],
                    help="a prompt of N seeded random token ids (repeat for a batch)")
    ap.add_argument("--no-graph", action="store_true", help="run decode steps kernel by kernel instead of replaying CUDA graphs")
    ap.add_argument("--stats-json", metavar="FILE", help="write the run's statistics as JSON to FILE ('-' = stdout)")
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


def print_top_k(logits_row, k: int, request: int, out=sys.stderr) -> None:
    """The reference's print_top_k_tokens (src/main.rs:165-207) for one row of logits."""
    import torch
    from .api import decode_bytes
    row = logits_row.detach().to(torch.float32).cpu()
    n_nan, n_inf = int(torch.isnan(row).sum()), int(torch.isinf(row).sum())
    if n_nan or n_inf:
        finite = row[torch.isfinite(row)]
        lo, hi, mean = (float(finite.min()), float(finite.max()), float(finite.mean())) if finite.numel() else (0.0, 0.0, 0.0)
        print(f"ERROR: logits of request {request} contain {n_nan} NaN and {n_inf} Inf values", file=out)
        print(f"  Stats: min={lo:.4f}, max={hi:.4f}, mean={mean:.4f}", file=out)
        return
    probs = torch.softmax(row.double(), dim=0)
    top = torch.topk(probs, min(k, row.numel()))
    print(f"Top-{len(top.indices)} tokens of request {request}:", file=out)
    for i, (p, idx) in enumerate(zip(top.values.tolist(), top.indices.tolist())):
        print(f"  {i + 1:2d}. {decode_bytes([idx])!r:10} ({p:.4f}) logit={float(row[idx]):.4f} id={idx}", file=out)


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
    if not args.prompt and not args.prompt_ids and not args.prompt_len:
        print("Error: --prompt <text>, --prompt-ids <ids> or --prompt-len <n> is required", file=sys.stderr)
        return 1
    try:
        from .engine.context import Options
        options = Options(decode_graphs=not args.no_graph)
        if args.model:
            llm = LLM(args.model, dtype=args.dtype, options=options)
        else:
            _, cfg = load_config(args.random_config)
            llm = LLM.random(cfg, args.random_seed, dtype=args.dtype, options=options)
        prompts = list(args.prompt) + [[int(t) for t in s.split(",") if t.strip()] for s in args.prompt_ids]
        gen = torch.Generator().manual_seed(args.random_seed)
        for n in args.prompt_len:
            prompts.append(torch.randint(0, llm.model.spec.vocab_size, (max(n, 1),), generator=gen).tolist())
        stops = None if args.stop_ids is None else [int(t) for t in args.stop_ids.split(",") if t.strip()]
        first = {}
        t0 = time.perf_counter()

        def on_token(i, tok):
            if i not in first:
                first[i] = time.perf_counter() - t0
            if args.debug:
                print(f"[Generated] request={i} token_id={tok}", file=sys.stderr)

        def on_logits(logits, requests, draws):
            # src/main.rs:725-727 (ten after the prompt), :954-957 (five for the tokens up to the third)
            for row, (r, d) in enumerate(zip(requests, draws)):
                if d <= 3:
                    print(f"\n[Token {d} logits]" if d else "\n[Prompt logits]", file=sys.stderr)
                    print_top_k(logits[row], 10 if d == 0 else 5, r)

        results = llm.generate(prompts, max_tokens=args.max_tokens, temperature=args.temperature,
                               top_p=args.top_p, top_k=args.top_k, seed=args.seed, stop_token_ids=stops,
                               on_token=on_token, on_logits=on_logits if args.debug else None)
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
    if args.stats_json:
        import json
        ttft = max(first.values()) if first else 0.0
        stats = {"requests": len(results), "prompt_tokens": n_prompt, "generated_tokens": n_gen,
                 "prefill_ms": ttft * 1e3, "prefill_tok_s": n_prompt / ttft if ttft > 0 else None,
                 "decode_ms": max(total - ttft, 0.0) * 1e3,
                 "decode_tok_s": n_gen / (total - ttft) if total > ttft else None,
                 "dtype": args.dtype, "graphs": not args.no_graph and not args.debug,
                 "results": [{"prompt_len": r.prompt_len, "tokens": len(r.tokens), "reason": r.reason} for r in results]}
        text = json.dumps(stats)
        if args.stats_json == "-":
            print(text)
        else:
            with open(args.stats_json, "w") as f:
                f.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
