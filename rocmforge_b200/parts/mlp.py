"""Gated feed-forward (SwiGLU)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..weights.spec import ParamSpec
from .base import FEED_FORWARDS, FeedForward
from .linear import Linear


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    """x += W_down (act(W_gate y) * (W_up y)), no biases
    (maeddesg/ROCmForge src/gpu/forward.rs:1094-1161, hip_kernels/elementwise.hip:72-82).

    gate and up are fused into one matrix at load time with their rows interleaved
    (row 2j = gate_j, row 2j+1 = up_j), so that one product yields both and the
    activation reads neighbouring columns (the reference fuses gate, up and SiLU in its
    decode kernels, src/gpu/forward.rs:2485-2500).
    """

    accepts_scaled_rows = True

    def __init__(self, hidden: int, intermediate: int, activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} has no kernel")
        self.hidden, self.intermediate = hidden, intermediate
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            "gate_proj.weight": ParamSpec((self.intermediate, self.hidden)),
            "up_proj.weight": ParamSpec((self.intermediate, self.hidden)),
            "down_proj.weight": ParamSpec((self.hidden, self.intermediate)),
        }

    def bind(self, params, compute_dtype):
        g, u = params["gate_proj.weight"], params["up_proj.weight"]
        gu = torch.stack([g, u], dim=1).reshape(2 * self.intermediate, self.hidden).contiguous()
        self.gate_up = Linear(gu)
        self.down = Linear(params["down_proj.weight"])

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def forward(self, ctx, y, stream):
        a = ctx.gated_activation(y, self.gate_up)                           # [T, I]
        self.down.add_to_stream(ctx, a, stream)
