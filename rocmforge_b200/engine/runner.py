"""The StepEngine of a real model: Model.step + the device sampler over one cache."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import kernels
from ..cache import pages_for
from ..sampling import DeviceSampler, SamplingParams
from .batch import StepRequest
from .generate import StepEngine


class ModelEngine(StepEngine):
    wants_final_hint = True          # ``run(..., final=True)``: no sequence of the call will be stepped again

    def __init__(self, model, cache, max_batch: int = 64):
        self.model = model
        self.cache = cache
        self.max_batch = max_batch
        self.max_seq_len = cache.max_seq_len
        self.sampler = DeviceSampler(model.device)
        self._calls = 0
        self._host_ids = None            # pinned buffer for the sampled ids
        self.logits_hook = None          # callable(logits [rows, vocab] on the device, requests, draws): the caller looks
                                         # at every step's logits; steps then run one by one, outside graphs
        self.decode_runner = None
        if model.options.decode_graphs:
            from .graph import DecodeRunner
            self.decode_runner = DecodeRunner(model, cache)

    def admit(self, prompt_lens: Sequence[int], max_new_tokens: int) -> int:
        free = min(self.cache.free_pages()) if self.cache.groups else 1 << 30
        slots = self.cache.slots.n_free
        n = 0
        for plen in prompt_lens:
            need = pages_for(min(plen + max_new_tokens, self.max_seq_len))
            if n >= self.max_batch or n >= slots or need > free:
                break
            free -= need
            n += 1
        return n

    def _to_host(self, out: torch.Tensor) -> List[int]:
        """The sampled ids on the host: through a pinned buffer, so that the copy is one call and one wait."""
        n = out.numel()
        if self._host_ids is None or self._host_ids.numel() < n or self._host_ids.dtype != out.dtype:
            self._host_ids = torch.empty((max(n, 64),), dtype=out.dtype).pin_memory()
            self._host_np = self._host_ids.numpy()
            self._host_done = torch.cuda.Event()
        self._host_ids[:n].copy_(out.reshape(-1), non_blocking=True)
        self._host_done.record()
        self._host_done.synchronize()
        return self._host_np[:n].tolist()

    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)
        if self.cache.live_slots == 0:     # a batch has ended: did any kernel give up waiting?
            kernels.tensor_core.check_status(self.model.device)

    def run(self, slots, tokens, requests, draws, sampling: SamplingParams, final: bool = False) -> List[int]:
        decode = all(len(t) == 1 for t in tokens)
        if decode and self.decode_runner is not None and self.logits_hook is None:
            # replayed from a graph with the sampler inside, one step ahead of the host
            ids = self.decode_runner.step_ids(slots, [t[0] for t in tokens], sampling, requests, draws, more=not final)
        else:
            if self.decode_runner is not None:
                self.decode_runner.drop_ahead()        # a step launched for sequences that all stopped
            reqs = [StepRequest(s, t, [len(t) - 1]) for s, t in zip(slots, tokens)]
            logits = self.model.step(self.cache, reqs)
            if self.logits_hook is not None:
                self.logits_hook(logits, list(requests), list(draws))
            ids = self._to_host(self.sampler.sample(logits, sampling, requests, draws))
        self._calls += 1
        if self._calls % 64 == 0:          # a separate small read: not on every step
            kernels.tensor_core.check_status(self.model.device)
        return ids
