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
from .stream import ScaledRows


@dataclass
class Options:
    """Switches of the engine (all default to the serving configuration)."""
    tensor_core_gemm: bool = True        # tcgen05 products on the bfloat16 path where the shape allows
    tuned_attention: bool = True         # split-KV decode attention / tiled prefill attention on bfloat16
    tcgen05_attention: bool = True       # prefill attention with tcgen05.mma (else the mma.sync kernel)
    clustered_decode: bool = True        # decode attention by clusters of CTAs (else one CTA per 128-key chunk)
    decode_graphs: bool = True           # replay decode steps from CUDA graphs in the generation loop
    # few tokens: the product that updates the stream also prepares the norm that follows (no norm kernel): its K splits
    # form a thread-block cluster and add their partial sums through shared memory.  Off: two kernels fewer a layer, but
    # the clusters start later than single CTAs do and end with two cluster barriers; measured per decode step, 7B shape:
    # batch 1 2.73 against 2.76 ms, batch 8 2.86 against 2.80 ms, batch 64 3.70 against 3.52 ms; 0.5B shape, batch 64:
    # 1.58 against 1.15 ms
    fused_norm: bool = False
    fused_norm_max_tokens: int = 32


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
        self.model_cache_limit = max_end     # inside a replayed graph: the longest sequence the cache holds
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
        known = {"tokens", "tok_seq", "tok_pos", "seq_slot", "seq_start", "seq_nnew", "cu_q", "want_rows", "seeds", "row_map"}
        self.tables = {name: v for name, v in views.items() if name not in known}      # the parts' own tables

    # ---------------------------------------------------------------- matrix products
    def uses_tensor_cores(self, x, w, mode) -> bool:
        return (self.compute_dtype == torch.bfloat16 and self.options.tensor_core_gemm
                and kernels.tensor_core.supported(x.shape[0], w.shape[0], w.shape[1], mode)
                and x.data_ptr() % 16 == 0 and (x.stride(0) * 2) % 16 == 0)

    def unpack_rows(self, x, w, mode):
        """(tensor, row_ss) of an activation: the sums of squares go along where the product scales rows itself,
        else the rows are normalised first."""
        if not isinstance(x, ScaledRows):
            return x, None
        tc = kernels.tensor_core
        if x.x.shape[0] <= tc.SKINNY_MAX_TOKENS and self.uses_tensor_cores(x.x, w, mode):
            return x.x, x.row_ss
        return x.materialize(), None

    def matmul(self, x, w, bias=None, *, out_f32=False):
        """x [M,K] @ w[N,K]^T (+ bias) -> [M,N] in the compute dtype, or in float32."""
        tc = kernels.tensor_core
        mode = tc.F32 if out_f32 else tc.STORE
        x, row_ss = self.unpack_rows(x, w, mode)
        if self.uses_tensor_cores(x, w, mode):
            if x.shape[0] <= tc.SKINNY_MAX_TOKENS:
                return tc.gemm_tc_skinny(x, w, bias, mode=mode, row_ss=row_ss)
            return tc.gemm_tc(x, w, bias, mode=mode)
        return kernels.gemm_simt(x, w, bias, out_f32=out_f32)

    def matmul_residual(self, x, w, bias, stream) -> None:
        """stream += x w^T (+ bias), summed in 32-bit: into ``h`` directly, or left pending as the
        32-bit partial sums of a K-split product (the next norm adds them in index order)."""
        tc = kernels.tensor_core
        follows = stream.take_hint()                 # the norm that reads the stream after this update, if we were told
        x, row_ss = self.unpack_rows(x, w, tc.RESIDUAL)
        if self.uses_tensor_cores(x, w, tc.RESIDUAL):
            if x.shape[0] <= tc.SKINNY_MAX_TOKENS:
                deferred = (follows.deferred_params() if (follows is not None and self.options.fused_norm
                                                          and x.shape[0] <= self.options.fused_norm_max_tokens) else None)
                if deferred is not None and deferred[0].shape == (w.shape[0],) and stream.h.is_contiguous():
                    # the split that finishes last adds all partial sums into the stream and prepares the norm
                    stream.flush()
                    normed, ss = tc.gemm_tc_skinny_resnorm(x, w, bias, stream.h, deferred[0],
                                                           splits=tc.resnorm_splits(w.shape[0], w.shape[1]), row_ss=row_ss)
                    stream.prepared = (follows, ScaledRows(normed, ss, deferred[1], w.shape[0]))
                    return
                splits = tc.split_k_for(w.shape[0], w.shape[1], tokens=x.shape[0]) if bias is None else 1
                if splits > 1:
                    stream.add_pending(tc.gemm_tc_skinny(x, w, mode=tc.PARTIAL, splits=splits, row_ss=row_ss))
                    return
                stream.flush()
                tc.gemm_tc_skinny(x, w, bias, mode=tc.RESIDUAL, out=stream.h, row_ss=row_ss)
                return
            stream.flush()
            tc.gemm_tc(x, w, bias, mode=tc.RESIDUAL, out=stream.h)
            return
        if x.shape[0] <= tc.SKINNY_MAX_TOKENS and bias is None:
            splits = kernels.split_k_for_simt(w.shape[0], w.shape[1])
            if splits > 1:                           # few tokens: K ranges in parallel, summed by the next norm
                stream.add_pending(kernels.gemm_simt(x, w, splits=splits))
                return
        stream.flush()
        kernels.gemm_simt(x, w, bias, out=stream.h, accumulate=True)

    def gated_activation(self, y, gate_up):
        """silu(gate) * up from the fused, row-interleaved gate/up matrix."""
        tc = kernels.tensor_core
        w = gate_up.weight
        y, row_ss = self.unpack_rows(y, w, tc.SWIGLU)
        if gate_up.bias is None and self.uses_tensor_cores(y, w, tc.SWIGLU):
            if y.shape[0] <= tc.SKINNY_MAX_TOKENS:
                return tc.gemm_tc_skinny(y, w, mode=tc.SWIGLU, row_ss=row_ss)
            return tc.gemm_tc(y, w, mode=tc.SWIGLU)
        if row_ss is not None:
            y = ScaledRows(y, row_ss[0], row_ss[1], w.shape[1]).materialize()
        gu = self.matmul(y, w, gate_up.bias)
        return kernels.swiglu(gu)
