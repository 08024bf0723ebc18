"""Rotary position encoding, NeoX pairing over the whole head."""
from __future__ import annotations

import torch

from .base import POSITIONS, PositionEncoding


@POSITIONS.register("rope_neox")
class NeoxRope(PositionEncoding):
    """Pairs (i, i + d/2) of a head are rotated by pos * theta^(-2i/d)
    (maeddesg/ROCmForge hip_kernels/rope.hip:57-90, src/cpu/ops.rs:69-98 with neox=true).

    ``rotary_dim`` (default: the whole head) limits the rotation to the first elements of a head, d then being
    ``rotary_dim``; ``interleaved`` pairs (2i, 2i+1) instead (the reference's neox=false branch, src/cpu/ops.rs:86-96).

    The reference evaluates powf in the kernel; here the d/2 frequencies are computed
    once in double precision, rounded to float32 and shared by every kernel, so that
    all of them (and the plain implementation) rotate by the same angle
    float32(pos) * float32(freq).
    """

    def __init__(self, head_dim: int, theta: float, rotary_dim: int = None, interleaved: bool = False):
        rot = head_dim if rotary_dim is None else int(rotary_dim)
        if head_dim % 2 or rot % 2 or not 0 < rot <= head_dim:
            raise ValueError(f"rotary encoding needs an even head_dim and an even rotary_dim in (0, head_dim]; "
                             f"got {head_dim} and {rot}")
        self.head_dim, self.rotary_dim, self.interleaved = head_dim, rot, bool(interleaved)
        self.theta = float(theta)
        i = torch.arange(rot // 2, dtype=torch.float64)
        self.inv_freq_host = (1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                              2.0 * i / rot)).to(torch.float32)
        self.inv_freq = None

    def prepare(self, device):
        self.inv_freq = self.inv_freq_host.to(device)

    def rotation(self):
        return dict(inv_freq=self.inv_freq, rot_dim=self.rotary_dim, interleaved=self.interleaved)
