"""Plain sampler and generation loop, restated from maeddesg/ROCmForge's
src/cpu/sampler.rs and src/main.rs; the oracle for the engine's sampler and loop.
It shares no code with ``rocmforge_b200``.
"""
from __future__ import annotations

import numpy as np
import torch

MASK64 = (1 << 64) - 1
REQUEST_STRIDE = 0x9E3779B97F4A7C15     # keeps the draws of two requests of a batch apart
DEFAULT_SEED = 0xDEADBEEF               # src/main.rs:739


def lcg_unit(seed: int) -> np.float32:
    """src/cpu/sampler.rs:180-185 — one multiply-add of a 64-bit LCG, top 53 bits,
    both operands of the division rounded to 32-bit floats."""
    v = (seed * 6364136223846793005 + 1442695040888963407) & MASK64
    return np.float32(np.float32(v >> 11) / np.float32(1 << 53))


def draw_seed(seed: int, request: int, draw: int) -> int:
    """The reference adds 1 to its seed before every draw (src/main.rs:747,979);
    a request's draws must not depend on its neighbours in a batch, so each
    request walks its own arithmetic sequence."""
    return (seed + 1 + draw + request * REQUEST_STRIDE) & MASK64


def greedy(logits: torch.Tensor) -> int:
    """argmax; of equal maxima the highest index wins (src/cpu/ops.rs:2244-2250,
    hip_kernels/elementwise.hip:154-155)."""
    x = logits.to(torch.float32)
    m = x.max()
    return int(torch.nonzero(x == m).max())


def sample(logits: torch.Tensor, temperature: float, top_p: float, top_k: int, seed: int) -> int:
    """Temperature, optional top-k, nucleus, one LCG draw
    (src/cpu/sampler.rs:22-71 top-p, :76-110 top-k, :115-177 both).

    Order of equal probabilities: lower index first (the reference's unstable sort
    leaves it open).  The exponentials are 32-bit as in the reference; the sums over them
    are taken in double precision: the reference's 32-bit running sums drop the tail of a
    large vocabulary (4.7e-4 of the mass at 152,064 entries), which no parallel sampler
    could or should reproduce.
    """
    if temperature == 0.0:                      # src/cli/chat.rs:483
        return greedy(logits)
    x = logits.to(torch.float32).numpy()
    t = np.float32(max(temperature, 1e-6))
    order = np.argsort(-x, kind="stable")       # descending value, ascending index among equals
    if top_k and top_k > 0:
        order = order[: min(top_k, len(order))]
    scaled = (x[order] / t).astype(np.float32)
    e = np.exp((scaled - scaled[0]).astype(np.float32)).astype(np.float32).astype(np.float64)
    probs = e / e.sum()
    cumsum = 0.0
    end = 1
    for i, p in enumerate(probs):
        cumsum += p
        end = i + 1
        if cumsum >= top_p:
            break
    rand_val = float(lcg_unit(seed)) * cumsum
    running = 0.0
    for i in range(end):
        running += probs[i]
        if running >= rand_val:
            return int(order[i])
    return int(order[0])


def generate(logits_fn, prompt, *, max_tokens, temperature=0.0, top_p=1.0, top_k=0,
             seed=DEFAULT_SEED, request=0, stop_ids=(), max_seq=None):
    """The reference's loop (src/main.rs:911-983) for one request, without a cache:
    ``logits_fn(tokens)`` returns the logits of the last position of ``tokens``.

    Returns (generated tokens, reason).  The stop token is not part of the output.
    """
    tokens = list(prompt)
    out = []
    draw = 0
    if max_tokens <= 0:
        return out, "max_tokens"
    while True:
        last = logits_fn(tokens)
        if temperature == 0.0:
            nxt = greedy(last)
        else:
            nxt = sample(last, temperature, top_p, top_k, draw_seed(seed, request, draw))
            draw += 1
        # order of the checks as in src/main.rs:913
        if nxt in stop_ids:
            return out, "stop_token"
        if max_seq is not None and len(tokens) >= max_seq:
            return out, "context_full"
        out.append(nxt)
        tokens.append(nxt)
        if len(out) >= max_tokens:
            return out, "max_tokens"
