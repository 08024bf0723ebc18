"""The residual stream of a step."""
from __future__ import annotations

from typing import Optional

import torch


class ScaledRows:
    """Activations whose rows still have to be divided by their RMS.

    ``x`` [T, H] is (residual stream * norm weight) in the compute dtype, ``ss`` [tiles, T] holds sums of squares of
    the stream per column tile; the normalised activations are x * rsqrt(sum_t ss[t] / width + eps) row by row.  A
    matrix product is linear in that factor, so a product that takes ``ScaledRows`` applies it to its output rows
    (in 32-bit, before bias and activation) and the norm never runs as a kernel of its own.
    """

    def __init__(self, x: torch.Tensor, ss: torch.Tensor, eps: float, width: int):
        self.x, self.ss, self.eps, self.width = x, ss, float(eps), int(width)
        self.shape = x.shape

    @property
    def row_ss(self):
        return (self.ss, self.eps)

    def materialize(self) -> torch.Tensor:
        """The normalised activations as an ordinary tensor (for a consumer that cannot scale rows itself)."""
        rstd = torch.rsqrt(self.ss.sum(dim=0) / self.width + self.eps)
        return (self.x.to(torch.float32) * rstd[:, None]).to(self.x.dtype)


class ResidualStream:
    """``h`` [T, H] in float32 plus one addend that has not been added yet.

    A part that produces an update either adds it into ``h`` itself (a matrix product whose
    epilogue accumulates) or leaves it as ``pending``: a [T, H] tensor of the compute dtype,
    or a float32 stack [S, T, H] of partial sums.  The next norm adds ``pending`` into ``h``
    in the same pass in which it normalises, which saves one read and one write of the
    stream per sub-layer.  The sum itself is always formed in 32-bit.

    ``next_norm`` is a hint from whoever arranges the parts (a block, the model): the norm that will read the stream
    after the next update.  A product that adds into ``h`` may take the hint and prepare that norm in its own
    epilogue; it then leaves the result in ``prepared`` = (norm, ScaledRows), which that norm hands on instead of
    launching.  Taking the hint is optional, and ``h`` is complete either way.
    """

    def __init__(self, h: torch.Tensor):
        self.h = h
        self.pending: Optional[torch.Tensor] = None
        self.next_norm = None
        self.after_block = None          # set by the model: the norm that reads the stream after this block
        self.prepared = None

    def add_pending(self, t: torch.Tensor) -> None:
        if self.pending is not None:
            self.flush()
        self.prepared = None             # the stream changes: what was prepared from it is stale
        self.next_norm = None
        self.pending = t

    def take_hint(self):
        """The norm that follows the update about to be made (or None); whatever was prepared before is dropped."""
        norm, self.next_norm = self.next_norm, None
        self.prepared = None
        return norm

    def flush(self) -> torch.Tensor:
        """Add what is pending into ``h`` now (a part that needs the up-to-date stream calls this)."""
        if self.pending is not None:
            p = self.pending
            p = p.sum(dim=0) if p.dim() == 3 else p.to(torch.float32)
            self.h.add_(p)
            self.pending = None
        return self.h
