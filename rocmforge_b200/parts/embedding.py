"""Token embedding and output head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..weights.spec import ParamSpec
from .base import Part
from .linear import Linear


class TokenEmbedding(Part):
    """x = E[token], no scaling (maeddesg/ROCmForge src/gpu/forward.rs:826-883)."""

    def __init__(self, vocab: int, hidden: int):
        self.vocab, self.hidden = vocab, hidden
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def bind(self, params, compute_dtype):
        self.weight = params["weight"]

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def forward(self, ctx, token_ids: torch.Tensor) -> torch.Tensor:
        return kernels.embed(self.weight, token_ids)


class OutputHead(Part):
    """logits = W y in float32; with tied embeddings W is the embedding matrix itself
    (maeddesg/ROCmForge src/gpu/forward.rs:1313-1338; tie: src/gpu/weights.rs:868-886)."""

    def __init__(self, vocab: int, hidden: int, tied_to: Optional[str] = None):
        self.vocab, self.hidden, self.tied_to = vocab, hidden, tied_to
        self.linear: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab, self.hidden), tied_to=self.tied_to)}

    def bind(self, params, compute_dtype):
        self.linear = Linear(params["weight"])

    def forward(self, ctx, y: torch.Tensor) -> torch.Tensor:
        return self.linear(ctx, y, out_f32=True)
