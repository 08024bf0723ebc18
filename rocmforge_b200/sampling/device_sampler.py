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
        self._pinned = None            # seeds on their way to the device: one pinned buffer, one copy a step
        self._pinned_np = None
        self._dev = None
        self._copied = None

    def _seeds(self, values) -> torch.Tensor:
        n = len(values)
        if self._pinned is None or self._pinned.numel() < n:
            cap = max(64, 2 * n)
            self._pinned = torch.zeros((cap,), dtype=torch.int64)
            if self.device.type == "cuda":
                self._pinned = self._pinned.pin_memory()
                self._copied = torch.cuda.Event()
            self._pinned_np = self._pinned.numpy()
            self._dev = torch.zeros((cap,), dtype=torch.int64, device=self.device)
            self._busy = False
        if self._copied is not None and self._busy:
            self._copied.synchronize()                     # the last copy may still read the pinned buffer
        self._pinned_np[:n] = values
        self._dev[:n].copy_(self._pinned[:n], non_blocking=True)
        if self._copied is not None:
            self._copied.record()
            self._busy = True
        return self._dev[:n]

    def sample(self, logits: torch.Tensor, params: SamplingParams, requests: Sequence[int],
               draws: Sequence[int], out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``requests[i]`` / ``draws[i]``: index of row i's request and of its draw, for the seed."""
        if params.greedy:
            return kernels.argmax(logits, out=out)
        seeds = self._seeds([as_int64(draw_seed(params.seed, r, d)) for r, d in zip(requests, draws)])
        return kernels.sample(logits, params.temperature, params.top_p, params.top_k, seeds, out=out)
