"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and owns no forward pass, cache or loader: it drives ``Model.step`` and
``SequenceCache``, the ones generation uses.  The nearest thing in maeddesg/ROCmForge are the
test helpers that push a prompt through token by token and keep the final logits
(tests/gpu_decode_real.rs:31-47).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step with wanted places the logits go to ``<out>/<step>.f32`` as little-endian
float32 [wanted, vocab], in the order of the entries and of ``want``.  After every step a
line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO

import numpy as np
import torch

from .. import kernels
from .batch import StepRequest


class TraceError(ValueError):
    pass


def replay(model, cache, lines: IO[str], out_dir: str, reply: IO[str] = sys.stdout) -> int:
    """Run every step read from ``lines``; returns the number of steps done."""
    os.makedirs(out_dir, exist_ok=True)
    slot_of: Dict[str, int] = {}
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        try:
            msg = json.loads(line)
        except json.JSONDecodeError as e:
            raise TraceError(f"trace line {n + 1} is not JSON: {e}") from None
        step = msg.get("step", n)
        entries = msg.get("entries", [])
        requests = []
        new_ids = []
        for e in entries:
            rid = str(e["id"])
            if rid not in slot_of:
                slot_of[rid] = cache.alloc_slot()
                new_ids.append(rid)
            requests.append(StepRequest(slot_of[rid], [int(t) for t in e["tokens"]],
                                        [int(w) for w in e.get("want", [])]))
        if requests:
            try:
                logits = model.step(cache, requests)
            except Exception:
                for rid in new_ids:                      # a refused step must not keep slots
                    cache.free_slot(slot_of.pop(rid))
                raise
            if logits is not None:
                arr = logits.detach().to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(out_dir, f"{step}.f32"))
            else:
                torch.cuda.synchronize(model.device)
            kernels.tensor_core.check_status(model.device)
        for rid in msg.get("end", []):
            rid = str(rid)
            if rid not in slot_of:
                raise TraceError(f"step {step}: request {rid!r} ends but never started")
            cache.free_slot(slot_of.pop(rid))
        reply.write(f"done {step}\n")
        reply.flush()
        n += 1
    return n


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    args = ap.parse_args(argv)

    from .model import Model
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is visible; this engine has no CPU path", file=sys.stderr)
        return 2
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    model = Model.from_folder(args.model, dtype=dtype, device="cuda:0")
    cache = model.new_cache(max_tokens=args.max_tokens)
    replay(model, cache, sys.stdin, args.out)
    return 0
