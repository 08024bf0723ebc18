"""What a part sees of the running step: the batch's device arrays and the kernel choices.

maeddesg/ROCmForge picks a kernel per weight type and environment flag in src/gpu/ops.rs
(gpu_dispatch_gemm :1591, gpu_dispatch_gemv :455) with switches cached from the
environment in src/gpu/safety.rs:34-66.  Here the choice depends on the compute dtype and
on the shape alone, and ``Options`` holds the few switches; there is never a fallback to
another device or to a library model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels


@dataclass
class Options:
    """Switches of the engine (all default to the serving configuration)."""
    tensor_core_gemm: bool = True        # tcgen05 products on the bfloat16 path where the shape allows
    tuned_attention: bool = True         # split-KV decode attention / tiled prefill attention on bfloat16
    decode_graphs: bool = True           # replay decode steps from CUDA graphs in the generation loop


class StepContext:
    """Device arrays of the batch and the kernel dispatch for one step."""

    def __init__(self, model, views, *, T: int, B: int, R: int, is_decode: bool, max_new: int, max_end: int,
                 host=None):
        self.model = model
        self.options: Options = model.options
        self.compute_dtype: torch.dtype = model.compute_dtype
        self.device = model.device
        self.T, self.B, self.R = T, B, R
        self.is_decode, self.max_new, self.max_end = is_decode, max_new, max_end
        self.host = host                     # the StepBatch (host arrays); None inside a replayed graph
        self.replayed = False                # True inside a CUDA graph: launch shapes must be fixed
        self.tokens = views["tokens"]
        self.tok_seq = views["tok_seq"]
        self.tok_pos = views["tok_pos"]
        self.seq_slot = views["seq_slot"]
        self.seq_start = views["seq_start"]
        self.seq_nnew = views["seq_nnew"]
        self.cu_q = views["cu_q"]
        self.want_rows = views["want_rows"]

    # ---------------------------------------------------------------- matrix products
    def matmul(self, x, w, bias=None, *, out_f32=False):
        return kernels.gemm_simt(x, w, bias, out_f32=out_f32)

    def matmul_residual(self, x, w, bias, stream) -> None:
        """stream.h += x w^T (+ bias), summed in 32-bit."""
        stream.flush()
        kernels.gemm_simt(x, w, bias, out=stream.h, accumulate=True)

    def gated_activation(self, y, gate_up):
        """silu(gate) * up from the fused, row-interleaved gate/up matrix."""
        gu = self.matmul(y, gate_up.weight, gate_up.bias)
        return kernels.swiglu(gu)

    # ---------------------------------------------------------------- attention
    def attention(self, qkv, mixer, view):
        """Attention of the step's tokens over the cache; q is the first heads*head_dim columns of ``qkv``."""
        return kernels.attention_generic(qkv, mixer.n_heads, mixer.n_kv_heads, mixer.head_dim,
                                         view.k_pages, view.v_pages, self.tok_seq, self.tok_pos,
                                         self.seq_slot, view.block_table, mixer.scale, view.window)
