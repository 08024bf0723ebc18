"""Picks next tokens from float32 logits on the device."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import kernels
from .params import SamplingParams, as_int64, draw_seed


class DeviceSampler:
    """Greedy rows go through the argmax kernel, the others through the sampling kernel;
    nothing but the chosen ids leaves the device.  maeddesg/ROCmForge samples on the host from
    downloaded logits and keeps only the argmax on the GPU (src/gpu/forward.rs:300-327)."""

    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: SamplingParams, requests: Sequence[int],
               draws: Sequence[int], out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``requests[i]`` / ``draws[i]``: index of row i's request and of its draw, for the seed."""
        if params.greedy:
            return kernels.argmax(logits, out=out)
        seeds = torch.tensor([as_int64(draw_seed(params.seed, r, d)) for r, d in zip(requests, draws)],
                             dtype=torch.int64).to(self.device, non_blocking=True)
        return kernels.sample(logits, params.temperature, params.top_p, params.top_k, seeds, out=out)
