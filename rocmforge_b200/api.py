"""The Python entry point: a model, its cache and the generation loop behind one object.

maeddesg/ROCmForge has no Python face; the option names (``max_tokens``, ``temperature``,
``top_p``) and their meanings are those of its command line (src/main.rs:42-66).
"""
from __future__ import annotations

import time
from typing import Iterable, List, Optional, Sequence, Union

import torch

from .engine.generate import GenerationResult, generate
from .engine.model import Model
from .engine.context import Options
from .engine.runner import ModelEngine
from .sampling import SamplingParams, DEFAULT_SEED

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def encode_bytes(text: str, vocab_size: int) -> List[int]:
    """Byte-level stand-in for a tokenizer: one id per UTF-8 byte."""
    ids = list(text.encode("utf-8"))
    if ids and max(ids) >= vocab_size:
        raise ValueError(f"the prompt holds byte {max(ids)}, the vocabulary has {vocab_size} ids")
    return ids


def decode_bytes(ids: Iterable[int]) -> str:
    out, run = [], bytearray()
    for i in ids:
        if 0 <= i < 256:
            run.append(i)
        else:
            if run:
                out.append(run.decode("utf-8", errors="replace"))
                run = bytearray()
            out.append(f"<{i}>")
    if run:
        out.append(run.decode("utf-8", errors="replace"))
    return "".join(out)


class LLM:
    """``LLM(model=folder)`` or ``LLM.random(config, seed)``; then ``generate(prompts, ...)``."""

    def __init__(self, model: Union[str, Model], dtype="bfloat16", device: str = "cuda:0",
                 cache_tokens: Optional[int] = None, max_batch: int = 64, options: Optional[Options] = None):
        if isinstance(model, Model):
            self.model = model
        else:
            self.model = Model.from_folder(model, dtype=_DTYPES[dtype], device=device, options=options)
        self.max_batch = max_batch
        self.cache_tokens = cache_tokens
        self.cache = None
        self.engine = None
        self.last_stats = {}

    @classmethod
    def random(cls, config, seed: int = 0, dtype="bfloat16", device: str = "cuda:0", **kw) -> "LLM":
        options = kw.pop("options", None)
        return cls(Model.random(config, seed, _DTYPES[dtype], device, options), **kw)

    def _ensure_cache(self, tokens_needed: int) -> None:
        want = self.cache_tokens or tokens_needed
        if self.cache is None or (self.cache_tokens is None and self.cache.n_pages * 64 < want):
            self.engine = None
            self.cache = None
            self.cache = self.model.new_cache(max_tokens=want)
            self.engine = ModelEngine(self.model, self.cache, max_batch=self.max_batch)

    def generate(self, prompts: Sequence[Union[str, Sequence[int]]], max_tokens: int = 256,
                 temperature: float = 1.0, top_p: float = 0.9, top_k: int = 0, seed: int = DEFAULT_SEED,
                 stop_token_ids: Optional[Iterable[int]] = None, on_token=None, on_logits=None) -> List[GenerationResult]:
        """Token ids in, token ids out (strings go through the byte-level stand-in tokenizer).

        ``on_logits(logits, requests, draws)`` sees the float32 logits (on the device) from which each step's tokens
        are drawn, row i belonging to request ``requests[i]`` at its ``draws[i]``-th token; steps then run one by one.

        ``temperature == 0`` decodes greedily.  Stop tokens default to the configuration's
        ``eos_token_id``; a stop token is not part of the output.
        """
        vocab = self.model.spec.vocab_size
        ids = [encode_bytes(p, vocab) if isinstance(p, str) else [int(t) for t in p] for p in prompts]
        for i, p in enumerate(ids):
            for t in p:
                if not 0 <= t < vocab:
                    raise ValueError(f"request {i}: token id {t} is outside the vocabulary of {vocab}")
        limit = self.model.spec.max_position
        per_seq = [min(len(p) + max_tokens, limit) for p in ids]
        batch = sorted(per_seq, reverse=True)[: self.max_batch]
        self._ensure_cache(sum((n + 63) // 64 * 64 for n in batch))
        stops = self.model.spec.stop_token_ids if stop_token_ids is None else stop_token_ids
        t0 = time.perf_counter()
        self.engine.logits_hook = on_logits
        try:
            out = generate(self.engine, ids, max_new_tokens=max_tokens,
                           sampling=SamplingParams(temperature, top_p, top_k, seed), stop_token_ids=stops,
                           on_token=on_token)
        finally:
            self.engine.logits_hook = None
        torch.cuda.synchronize(self.model.device)
        dt = time.perf_counter() - t0
        n_out = sum(len(r.tokens) for r in out)
        self.last_stats = {"seconds": dt, "generated": n_out, "tokens_per_second": n_out / dt if dt > 0 else 0.0}
        return out
