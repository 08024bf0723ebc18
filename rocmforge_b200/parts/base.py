"""Interfaces of the parts a model is put together from, and their registries.

A model is a list of blocks; a block arranges a mixer, a feed-forward and norms; a mixer
may use a position encoding.  Every part gets its sizes and constants as constructor
parameters and never learns which model it sits in; which part a layer uses is data
(a kind name and parameters) chosen by the architecture's builder from its configuration.

maeddesg/ROCmForge hard-wires one layer function per phase (src/gpu/forward.rs:886-1195 for
prefill, :2327-2534 for decode) whose kernels take eps, theta, head counts and head_dim
as arguments (hip_kernels/rope.hip:48-56, norm.hip:18-24); the parts below carry the same
constants, and one ``forward`` serves both phases.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from ..weights.spec import ParamSpec


class Part:
    """Something with named tensors.

    ``param_specs`` gives the local names (joined to the part's prefix by the model),
    ``bind`` receives the loaded tensors under the same local names, and
    ``cuda_modules`` names the CUDA modules the part launches for a compute dtype.
    """

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, params: Dict[str, torch.Tensor], compute_dtype: torch.dtype) -> None:
        pass

    def cuda_modules(self, compute_dtype: torch.dtype) -> List[str]:
        return []

    def step_table_names(self):
        """Names of int32 tables that this part builds on the host for every step (``step_table``).  They travel with
        the step descriptor in its one copy and reach the part as ``ctx.tables[name]``.  A name identifies its
        content: of several parts that name the same table, the first one builds it for all."""
        return ()

    def step_table(self, name: str, batch):
        """The table ``name`` for ``batch`` (an engine.batch.StepBatch: B, n_new, starts, is_decode, ...)."""
        raise NotImplementedError


class Norm(Part):
    """y = norm(h + pending).  See engine.stream.ResidualStream for ``stream``.

    ``deferred_ok``: the caller's consumer takes ``engine.stream.ScaledRows`` (rows not yet divided by their RMS)
    as well as a tensor; a norm that was prepared by the product before it may then hand those on.
    ``deferred_params`` returns (weight, eps) if the norm is y = x * rsqrt(mean(x^2) + eps) * weight, so that a
    product can prepare it in its epilogue, else None.
    """

    def forward(self, ctx, stream, rows: Optional[torch.Tensor] = None, deferred_ok: bool = False):
        raise NotImplementedError

    def deferred_params(self):
        return None


class PositionEncoding(Part):
    """Knows how a position changes queries and keys; used by mixers that want one.

    ``rotation()`` is what the encoding hands to the kernel that rotates queries and keys on their way into the
    cache: a dict with ``inv_freq`` (float32 [rot_dim/2] on the device, pair i turns by position * inv_freq[i]),
    ``rot_dim`` (how many leading elements of a head turn; the rest pass through) and ``interleaved`` (pairs
    (2i, 2i+1) instead of (i, i + rot_dim/2)).  An encoding that does not rotate returns None (a mixer built with
    ``position=None`` behaves the same): queries and keys then go into the cache as they are.
    """

    def prepare(self, device) -> None:
        pass

    def rotation(self):
        return None


class Mixer(Part):
    """Mixes information between the positions of a sequence (attention here).

    ``cache_request`` says what the mixer keeps per sequence: a ``KVRequest``, a
    ``StateRequest`` or None.  ``forward`` gets the normed activations ``y`` [T, H]
    of the step's tokens, the view of its cache, and adds its result to ``stream``.
    """

    accepts_scaled_rows = False      # True: ``y`` may be an engine.stream.ScaledRows (passed on to ctx's products)

    def cache_request(self):
        return None

    def forward(self, ctx, y: torch.Tensor, cache_view, stream) -> None:
        raise NotImplementedError


class FeedForward(Part):
    """Position-wise transformation (dense here; routed experts would live behind the same face)."""

    accepts_scaled_rows = False      # as for Mixer

    def forward(self, ctx, y: torch.Tensor, stream) -> None:
        raise NotImplementedError


class Block(Part):
    """Arrangement of norm(s), mixer and feed-forward around the residual stream."""

    mixer: Mixer

    def forward(self, ctx, stream, cache_view) -> None:
        raise NotImplementedError

    def entry_norm(self):
        """The norm that reads the stream first when this block runs, if the block lets the product before it
        prepare that norm (see ResidualStream.next_norm); None otherwise."""
        return None

    def sub_parts(self) -> Dict[str, Part]:
        """{prefix relative to the block: part}."""
        raise NotImplementedError


# --------------------------------------------------------------------------- registries

class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: Dict[str, Callable] = {}

    def register(self, kind: str, factory: Callable = None):
        def deco(f):
            self._kinds[kind] = f
            return f
        return deco(factory) if factory is not None else deco

    def build(self, kind: str, **params):
        if kind not in self._kinds:
            raise KeyError(f"no {self.what} of kind {kind!r} is registered (known: {sorted(self._kinds)})")
        return self._kinds[kind](**params)

    def kinds(self):
        return sorted(self._kinds)


NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
