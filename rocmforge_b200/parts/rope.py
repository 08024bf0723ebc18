"""Rotary position encoding, NeoX pairing over the whole head."""
from __future__ import annotations

import torch

from .base import POSITIONS, PositionEncoding


@POSITIONS.register("rope_neox")
class NeoxRope(PositionEncoding):
    """Pairs (i, i + d/2) of a head are rotated by pos * theta^(-2i/d)
    (maeddesg/ROCmForge hip_kernels/rope.hip:57-90, src/cpu/ops.rs:69-98 with neox=true).

    The reference evaluates powf in the kernel; here the d/2 frequencies are computed
    once in double precision, rounded to float32 and shared by every kernel, so that
    all of them (and the plain implementation) rotate by the same angle
    float32(pos) * float32(freq).
    """

    def __init__(self, head_dim: int, theta: float):
        if head_dim % 2:
            raise ValueError("rotary encoding needs an even head_dim")
        self.head_dim = head_dim
        self.theta = float(theta)
        i = torch.arange(head_dim // 2, dtype=torch.float64)
        self.inv_freq_host = (1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                              2.0 * i / head_dim)).to(torch.float32)
        self.inv_freq = None

    def prepare(self, device):
        self.inv_freq = self.inv_freq_host.to(device)
