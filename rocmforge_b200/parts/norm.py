"""RMSNorm fused with the pending residual add."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..weights.spec import ParamSpec
from .base import NORMS, Norm


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """y_i = x_i * rsqrt(mean(x^2) + eps) * w_i, sums and rsqrt in 32-bit; the weight multiplies
    after normalisation and is used as stored (no 1 + w)
    (maeddesg/ROCmForge hip_kernels/norm.hip:18-84, src/cpu/ops.rs:32-46)."""

    def __init__(self, size: int, eps: float):
        self.size = size
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None
        self.compute_dtype = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), kind="vector", init="ones")}

    def bind(self, params, compute_dtype):
        self.weight = params["weight"]
        self.compute_dtype = compute_dtype

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def deferred_params(self):
        return (self.weight, self.eps)

    def forward(self, ctx, stream, rows=None, deferred_ok=False):
        prepared, stream.prepared = stream.prepared, None
        if prepared is not None and prepared[0] is self and rows is None and stream.pending is None:
            # the product that updated the stream has multiplied by this norm's weight and left the sums of squares
            return prepared[1] if deferred_ok else prepared[1].materialize()
        y = kernels.add_rmsnorm(stream.h, self.weight, self.eps, self.compute_dtype,
                                pending=stream.pending, rows=rows)
        if rows is None:
            stream.pending = None           # the kernel added it into h
        return y
