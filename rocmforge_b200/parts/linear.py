"""y = x W^T (+ bias): chooses the matrix-product kernel for a shape and a dtype."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels


class Linear:
    """A weight [N, K] (and an optional bias [N]) with the ways a part may apply it.

    On the float32 path every product runs on CUDA cores with 32-bit operands and sums.
    On the bfloat16 path the tensor-core kernels are used where the shape allows and the
    CUDA-core kernel otherwise; both accumulate in 32-bit.
    """

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.weight = weight
        self.bias = bias
        self.N, self.K = weight.shape

    def __call__(self, ctx, x: torch.Tensor, *, out_f32: bool = False) -> torch.Tensor:
        """x [M, K] -> [M, N] in the compute dtype (or float32)."""
        return ctx.matmul(x, self.weight, self.bias, out_f32=out_f32)

    def add_to_stream(self, ctx, x: torch.Tensor, stream) -> None:
        """stream += x W^T: the product lands in the residual stream, in 32-bit."""
        ctx.matmul_residual(x, self.weight, self.bias, stream)
