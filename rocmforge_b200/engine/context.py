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
    # few tokens: the product that updates the stream also prepares the norm that follows (no norm kernel).  Off: at
    # the 7B shape the split that finishes an output tile last needs as long for the fence, the counter and the partial
    # sums of its tile (o product 6.3 -> 11.0 us, down 22.9 -> 25.9 us at batch 8) as the two norm kernels took
    # (7.6 us a layer): 2.92 ms a step against 2.91 ms; with 64 tokens, or the 19 splits of the 0.5B shape, it loses
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
        self.q_tiles = views["q_tiles"]
        self.q_tiles128 = views["q_tiles128"]

    # ---------------------------------------------------------------- matrix products
    def _tensor_cores(self, x, w, mode) -> bool:
        return (self.compute_dtype == torch.bfloat16 and self.options.tensor_core_gemm
                and kernels.tensor_core.supported(x.shape[0], w.shape[0], w.shape[1], mode)
                and x.data_ptr() % 16 == 0 and (x.stride(0) * 2) % 16 == 0)

    def _rows(self, x, w, mode):
        """(tensor, row_ss) of an activation: the sums of squares go along where the product scales rows itself,
        else the rows are normalised first."""
        if not isinstance(x, ScaledRows):
            return x, None
        tc = kernels.tensor_core
        if x.x.shape[0] <= tc.SKINNY_MAX_TOKENS and self._tensor_cores(x.x, w, mode):
            return x.x, x.row_ss
        return x.materialize(), None

    def matmul(self, x, w, bias=None, *, out_f32=False):
        """x [M,K] @ w[N,K]^T (+ bias) -> [M,N] in the compute dtype, or in float32."""
        tc = kernels.tensor_core
        mode = tc.F32 if out_f32 else tc.STORE
        x, row_ss = self._rows(x, w, mode)
        if self._tensor_cores(x, w, mode):
            if x.shape[0] <= tc.SKINNY_MAX_TOKENS:
                return tc.gemm_tc_skinny(x, w, bias, mode=mode, row_ss=row_ss)
            return tc.gemm_tc(x, w, bias, mode=mode)
        return kernels.gemm_simt(x, w, bias, out_f32=out_f32)

    def matmul_residual(self, x, w, bias, stream) -> None:
        """stream += x w^T (+ bias), summed in 32-bit: into ``h`` directly, or left pending as the
        32-bit partial sums of a K-split product (the next norm adds them in index order)."""
        tc = kernels.tensor_core
        follows = stream.take_hint()                 # the norm that reads the stream after this update, if we were told
        x, row_ss = self._rows(x, w, tc.RESIDUAL)
        if self._tensor_cores(x, w, tc.RESIDUAL):
            if x.shape[0] <= tc.SKINNY_MAX_TOKENS:
                deferred = (follows.deferred_params() if (follows is not None and self.options.fused_norm
                                                          and x.shape[0] <= self.options.fused_norm_max_tokens) else None)
                if deferred is not None and deferred[0].shape == (w.shape[0],) and stream.h.is_contiguous():
                    # the split that finishes last adds all partial sums into the stream and prepares the norm
                    stream.flush()
                    normed, ss = tc.gemm_tc_skinny_resnorm(x, w, bias, stream.h, deferred[0],
                                                           splits=tc.split_k_for(w.shape[0], w.shape[1]), row_ss=row_ss)
                    stream.prepared = (follows, ScaledRows(normed, ss, deferred[1], w.shape[0]))
                    return
                splits = tc.split_k_for(w.shape[0], w.shape[1]) if bias is None else 1
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
        y, row_ss = self._rows(y, w, tc.SWIGLU)
        if gate_up.bias is None and self._tensor_cores(y, w, tc.SWIGLU):
            if y.shape[0] <= tc.SKINNY_MAX_TOKENS:
                return tc.gemm_tc_skinny(y, w, mode=tc.SWIGLU, row_ss=row_ss)
            return tc.gemm_tc(y, w, mode=tc.SWIGLU)
        if row_ss is not None:
            y = ScaledRows(y, row_ss[0], row_ss[1], w.shape[1]).materialize()
        gu = self.matmul(y, w, gate_up.bias)
        return kernels.swiglu(gu)

    # ---------------------------------------------------------------- attention
    def project_qkv_into_cache(self, y, mixer, view):
        """q/k/v projection (+ bias), rotation, cache write; returns rotated q [T, >= heads*head_dim].

        With few tokens on the tensor-core path the product is K-split for parallelism and the
        rotation kernel sums the 32-bit partial sums (and the bias) itself, so q/k/v never
        exist as an intermediate bfloat16 tensor.
        """
        tc = kernels.tensor_core
        w, bias = mixer.qkv.weight, mixer.qkv.bias
        y, row_ss = self._rows(y, w, tc.PARTIAL)
        rot = dict((mixer.position.rotation() if mixer.position is not None else None) or dict(inv_freq=None, rot_dim=0))
        inv_freq = rot.pop("inv_freq")
        rope = dict(rot_dim=rot["rot_dim"], interleaved=rot.get("interleaved", False), tok_seq=self.tok_seq, tok_pos=self.tok_pos, seq_slot=self.seq_slot,
                    block_table=view.block_table, k_pages=view.k_pages, v_pages=view.v_pages, write_kv=view.writes)
        if y.shape[0] <= tc.SKINNY_MAX_TOKENS and self._tensor_cores(y, w, tc.PARTIAL):
            splits = tc.split_k_for(w.shape[0], w.shape[1])
            if splits > 1:
                parts = tc.gemm_tc_skinny(y, w, mode=tc.PARTIAL, splits=splits, row_ss=row_ss)
                return kernels.rope_kv_write(parts, mixer.n_heads, mixer.n_kv_heads, mixer.head_dim,
                                             inv_freq, bias=bias, compute_dtype=self.compute_dtype,
                                             **rope)
        if row_ss is not None:
            y = ScaledRows(y, row_ss[0], row_ss[1], w.shape[1])
        elif y.shape[0] <= tc.SKINNY_MAX_TOKENS and not self._tensor_cores(y, w, tc.STORE):
            splits = kernels.split_k_for_simt(w.shape[0], w.shape[1])
            if splits > 1:                           # CUDA-core product of few tokens: the same scheme
                parts = kernels.gemm_simt(y, w, splits=splits)
                return kernels.rope_kv_write(parts, mixer.n_heads, mixer.n_kv_heads, mixer.head_dim,
                                             inv_freq, bias=bias, compute_dtype=self.compute_dtype,
                                             **rope)
        qkv = self.matmul(y, w, bias)
        return kernels.rope_kv_write(qkv, mixer.n_heads, mixer.n_kv_heads, mixer.head_dim,
                                     inv_freq, **rope)

    def attention(self, q, mixer, view):
        """Attention of the step's tokens over the cache; q is the first heads*head_dim columns of ``q``."""
        nh, nkv, hd = mixer.n_heads, mixer.n_kv_heads, mixer.head_dim
        longest = self.model_cache_limit if self.replayed else self.max_end
        if (self.is_decode and self.compute_dtype == torch.bfloat16 and self.options.tuned_attention
                and kernels.attention_decode_supported(nh, nkv, hd)):
            if self.options.clustered_decode:
                # a cluster of 1..8 CTAs per (sequence, kv head), every warp on its own tiles of keys, merged
                # through distributed shared memory: no scratch memory, no second pass, any context length
                return kernels.attention_decode_warps(
                    q, nh, nkv, hd, view.k_pages, view.v_pages, self.tok_seq, self.tok_pos, self.seq_slot,
                    view.block_table, mixer.scale, view.window,
                    splits=kernels.decode_splits(self.B, nkv, longest, view.window))
            if longest <= kernels.DECODE_CHUNK * kernels.DECODE_CHUNK:
                # the earlier kernel: one CTA per 128-key chunk, partial results merged through scratch memory
                need = max(1, (longest + kernels.DECODE_CHUNK - 1) // kernels.DECODE_CHUNK)
                max_chunks = 1
                while max_chunks < need:                   # powers of two: few distinct scratch sizes
                    max_chunks *= 2
                cap = 1
                while cap < self.B:
                    cap *= 2
                n_o, n_ml, n_c = kernels.attention_decode_scratch(cap, nh, nkv, hd, max_chunks)
                scratch = self.model.scratch
                return kernels.attention_decode(
                    q, nh, nkv, hd, view.k_pages, view.v_pages, self.tok_seq, self.tok_pos, self.seq_slot,
                    view.block_table, mixer.scale, view.window, max_chunks,
                    scratch("attn_decode_o", n_o, torch.float32), scratch("attn_decode_ml", n_ml, torch.float32),
                    kernels.tensor_core.register_counters(scratch("attn_decode_counters", n_c, torch.int32)))
        if (not self.is_decode and self.compute_dtype == torch.bfloat16 and self.options.tuned_attention
                and self.options.tcgen05_attention and self.q_tiles128.numel() > 0
                and kernels.attention_prefill_tc_supported(nh, nkv, hd)
                and q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0):
            return kernels.attention_prefill_tc(q, nh, nkv, hd, view.k_pages, view.v_pages, self.q_tiles128,
                                                self.seq_slot, self.seq_start, self.seq_nnew, self.cu_q,
                                                view.block_table, mixer.scale, view.window)
        if (not self.is_decode and self.compute_dtype == torch.bfloat16 and self.options.tuned_attention
                and self.q_tiles.numel() > 0 and kernels.attention_prefill_supported(nh, nkv, hd)
                and q.data_ptr() % 4 == 0 and q.stride(0) % 2 == 0):
            return kernels.attention_prefill(q, nh, nkv, hd, view.k_pages, view.v_pages, self.q_tiles, self.seq_slot,
                                             self.seq_start, self.seq_nnew, self.cu_q, view.block_table, mixer.scale,
                                             view.window)
        return kernels.attention_generic(q, nh, nkv, hd, view.k_pages, view.v_pages, self.tok_seq, self.tok_pos,
                                         self.seq_slot, view.block_table, mixer.scale, view.window)
