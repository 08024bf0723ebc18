"""The residual stream of a step."""
from __future__ import annotations

from typing import Optional

import torch


class ResidualStream:
    """``h`` [T, H] in float32 plus one addend that has not been added yet.

    A part that produces an update either adds it into ``h`` itself (a matrix product whose
    epilogue accumulates) or leaves it as ``pending``: a [T, H] tensor of the compute dtype,
    or a float32 stack [S, T, H] of partial sums.  The next norm adds ``pending`` into ``h``
    in the same pass in which it normalises, which saves one read and one write of the
    stream per sub-layer.  The sum itself is always formed in 32-bit.
    """

    def __init__(self, h: torch.Tensor):
        self.h = h
        self.pending: Optional[torch.Tensor] = None

    def add_pending(self, t: torch.Tensor) -> None:
        if self.pending is not None:
            self.flush()
        self.pending = t

    def flush(self) -> torch.Tensor:
        """Add what is pending into ``h`` now (a part that needs the up-to-date stream calls this)."""
        if self.pending is not None:
            p = self.pending
            p = p.sum(dim=0) if p.dim() == 3 else p.to(torch.float32)
            self.h.add_(p)
            self.pending = None
        return self.h
