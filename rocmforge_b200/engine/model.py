"""A model put together from parts, and its one step function.

``ModelSpec`` is what an architecture's builder returns: the parts, their tensor-name
prefixes and the order in which layers run.  ``Model`` binds weights to it and steps
batches through it.  The step is the counterpart of maeddesg/ROCmForge's
gpu_prefill_forward_hybrid (src/gpu/forward.rs:1198-1393) and gpu_full_forward_hybrid
(:2589-2745) in one function: it runs exactly the tokens it is given, reads everything
earlier from the cache, and returns float32 logits for the wanted rows.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import SequenceCache
from ..parts.base import Block, Norm, Part
from ..parts.embedding import OutputHead, TokenEmbedding
from ..weights import ParamSpec, load_folder, random_tensors
from .batch import BatchError, DeviceDescriptor, StepBatch, StepRequest
from .context import Options, StepContext
from .stream import ResidualStream


@dataclass
class ScheduleEntry:
    """One execution of a layer.  ``kv_from``: index of an earlier schedule entry whose cache
    this execution reads instead of keeping its own (it then writes nothing)."""
    layer: int
    kv_from: Optional[int] = None


@dataclass
class ModelSpec:
    config: object
    embedding: TokenEmbedding
    embedding_prefix: str
    blocks: List[Block]
    block_prefixes: List[str]
    final_norm: Norm
    final_norm_prefix: str
    head: OutputHead
    head_prefix: str
    schedule: List[ScheduleEntry]
    vocab_size: int
    hidden_size: int
    max_position: int
    stop_token_ids: List[int] = field(default_factory=list)

    def named_parts(self) -> Dict[str, Part]:
        """{tensor-name prefix: leaf part}."""
        out: Dict[str, Part] = {self.embedding_prefix: self.embedding}
        for prefix, block in zip(self.block_prefixes, self.blocks):
            for sub, part in block.sub_parts().items():
                out[prefix + sub] = part
        out[self.final_norm_prefix] = self.final_norm
        out[self.head_prefix] = self.head
        return out

    def param_specs(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for prefix, part in self.named_parts().items():
            for local, spec in part.param_specs().items():
                out[prefix + local] = spec
        return out

    def cache_requests(self) -> Dict[int, object]:
        """{schedule index: what that execution's mixer keeps per sequence}."""
        out = {}
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {e.layer}; there are {len(self.blocks)}")
            if e.kv_from is not None:
                if not 0 <= e.kv_from < i or self.schedule[e.kv_from].kv_from is not None:
                    raise ValueError(f"schedule entry {i}: kv_from must name an earlier entry that owns a cache")
                continue
            out[i] = self.blocks[e.layer].mixer.cache_request()
        return out

    def cuda_modules(self, compute_dtype) -> List[str]:
        mods: List[str] = ["gemm_simt", "sampling"]
        if compute_dtype == torch.bfloat16:
            mods.append("gemm_tcgen05")
            from ..csrc import build
            if build.available("gemm_tcgen05_cluster"):
                mods.append("gemm_tcgen05_cluster")
        for part in self.named_parts().values():
            mods += part.cuda_modules(compute_dtype)
        return list(dict.fromkeys(mods))


class Model:
    """Weights bound to a ModelSpec on one CUDA device."""

    def __init__(self, spec: ModelSpec, params: Dict[str, torch.Tensor], compute_dtype: torch.dtype, device,
                 options: Optional[Options] = None):
        from ..csrc import build
        self.spec = spec
        self.config = spec.config
        self.compute_dtype = compute_dtype
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("rocmforge_b200 models run on a CUDA device only (there is no CPU fallback)")
        self.options = options or Options()
        build.ensure_built(spec.cuda_modules(compute_dtype))
        for prefix, part in spec.named_parts().items():
            local = {name[len(prefix):]: t for name, t in params.items()
                     if name.startswith(prefix) and name[len(prefix):] in part.param_specs()}
            part.bind(local, compute_dtype)
        self._tables = {}                  # name -> builder of a host table that a part wants with every step
        for part in spec.named_parts().values():
            for name in part.step_table_names():
                self._tables.setdefault(name, (lambda batch, part=part, name=name: part.step_table(name, batch)))
        self._desc = DeviceDescriptor(self.device)
        self._scratch: Dict[tuple, torch.Tensor] = {}
        self.weight_bytes = sum(t.numel() * t.element_size()
                                for t in {t.data_ptr(): t for t in params.values()}.values())

    # ---------------------------------------------------------------- construction
    @classmethod
    def from_folder(cls, folder: str, dtype=torch.bfloat16, device="cuda:0", options=None) -> "Model":
        from ..config import load_config
        arch, config = load_config(folder)
        spec = arch.build(config)
        params = load_folder(folder, spec.param_specs(), dtype, device)
        return cls(spec, params, dtype, device, options)

    @classmethod
    def random(cls, config, seed: int = 0, dtype=torch.bfloat16, device="cuda:0", options=None) -> "Model":
        """Random weights made on the device (nothing is written to disk)."""
        from ..config import architecture_for
        from ..weights.loader import target_dtype
        spec = architecture_for(config.architecture).build(config)
        specs = spec.param_specs()
        params = {}
        for name, t in random_tensors(specs, seed, dtype, device):
            params[name] = t.to(target_dtype(specs[name], t.dtype, dtype))
        for name, s in specs.items():
            if name not in params:
                params[name] = params[s.tied_to]
        return cls(spec, params, dtype, device, options)

    def scratch(self, name: str, n: int, dtype: torch.dtype) -> torch.Tensor:
        """Zero-initialised scratch memory that kernels share from launch to launch.  A buffer, once handed
        out, is never freed or moved (captured graphs keep its address); a larger request gets a new one."""
        key = (name, n, dtype)
        if key not in self._scratch:
            self._scratch[key] = torch.zeros((max(n, 1),), dtype=dtype, device=self.device)
        return self._scratch[key]

    # ---------------------------------------------------------------- cache
    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None) -> SequenceCache:
        return SequenceCache(self.spec.cache_requests(), max_tokens=max_tokens, max_slots=max_slots,
                             max_seq_len=self.spec.max_position, dtype=self.compute_dtype, device=self.device)

    # ---------------------------------------------------------------- the step
    def step(self, cache: SequenceCache, requests: Sequence[StepRequest]) -> Optional[torch.Tensor]:
        """Run the given tokens of each request from the cache; float32 logits [wanted rows, vocab]
        in the order of the requests and of their ``want`` lists (None if nothing is wanted)."""
        requests = [r if isinstance(r, StepRequest) else StepRequest(*r) for r in requests]
        slots = [r.slot for r in requests]
        n_new = [len(r.tokens) for r in requests]
        for r in requests:
            if len(r.tokens) == 0:
                raise BatchError(f"slot {r.slot}: a step must bring at least one token")
        # build (and validate) the batch before any page is taken
        starts_now = [cache.length(s) if cache.slots.is_held(s) else 0 for s in slots]
        batch = StepBatch(requests, starts_now, self.spec.vocab_size, tables=self._tables)
        cache.prepare(slots, n_new)
        try:
            self._desc.upload(batch.pack())
            views = self._desc.views(batch.T, batch.B, batch.R, batch.extras)
            ctx = StepContext(self, views, T=batch.T, B=batch.B, R=batch.R, is_decode=batch.is_decode,
                              max_new=batch.max_new, max_end=batch.max_end, host=batch)
            logits = self.forward(ctx, cache)
        except BaseException:
            cache.rollback(slots)          # a step that did not happen keeps no pages
            raise
        cache.commit(slots, n_new)
        return logits

    def forward(self, ctx: StepContext, cache: SequenceCache) -> Optional[torch.Tensor]:
        """The layers in schedule order on the batch that ``ctx`` describes."""
        spec = self.spec
        stream = ResidualStream(spec.embedding.forward(ctx, ctx.tokens))
        for i, entry in enumerate(spec.schedule):
            owner = i if entry.kv_from is None else entry.kv_from
            view = cache.view(owner, writes=entry.kv_from is None)
            # the norm that reads the stream after this block: the next execution's first norm (the final norm gathers
            # rows and runs as a kernel of its own)
            nxt = spec.schedule[i + 1] if i + 1 < len(spec.schedule) else None
            stream.after_block = spec.blocks[nxt.layer].entry_norm() if nxt is not None else None
            spec.blocks[entry.layer].forward(ctx, stream, view)
        stream.next_norm = stream.after_block = None
        if ctx.R == 0:
            return None
        y = spec.final_norm.forward(ctx, stream, rows=ctx.want_rows)
        return spec.head.forward(ctx, y)
