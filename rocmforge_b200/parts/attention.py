"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

from .. import kernels
from ..cache.requests import KVRequest
from ..engine.stream import ScaledRows
from ..weights.spec import ParamSpec
from .base import MIXERS, Mixer, POSITIONS
from .linear import Linear


@MIXERS.register("gqa_attention")
class GQAAttention(Mixer):
    """q/k/v projections (with or without bias), rotation of q and k, write of k and v into
    the cache, softmax attention of the new tokens over the cache, output projection.

    Order and formulas follow maeddesg/ROCmForge src/gpu/forward.rs:940-1079 (prefill) and
    :2361-2472 (decode): the bias is added after the product and before the rotation;
    head h reads kv head h // (heads / kv_heads); scores are scaled by 1/sqrt(head_dim)
    (forward.rs:583); a query at position p sees keys 0..=p, or the last ``window`` of them.
    The three projections are fused into one matrix at load time (the reference fuses them
    in its decode kernels, src/gpu/ops.rs:748-880).
    """

    accepts_scaled_rows = True

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, *, qkv_bias: bool,
                 o_bias: bool = False, window: Optional[int] = None, position=None,
                 scale: Optional[float] = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} kv heads")
        self.hidden, self.n_heads, self.n_kv_heads, self.head_dim = hidden, n_heads, n_kv_heads, head_dim
        self.qkv_bias, self.o_bias, self.window = qkv_bias, o_bias, window
        self.position = position
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.q_size = n_heads * head_dim
        self.kv_size = n_kv_heads * head_dim
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        s = {
            "q_proj.weight": ParamSpec((self.q_size, self.hidden)),
            "k_proj.weight": ParamSpec((self.kv_size, self.hidden)),
            "v_proj.weight": ParamSpec((self.kv_size, self.hidden)),
            "o_proj.weight": ParamSpec((self.hidden, self.q_size)),
        }
        if self.qkv_bias:
            s["q_proj.bias"] = ParamSpec((self.q_size,), kind="vector")
            s["k_proj.bias"] = ParamSpec((self.kv_size,), kind="vector")
            s["v_proj.bias"] = ParamSpec((self.kv_size,), kind="vector")
        if self.o_bias:
            s["o_proj.bias"] = ParamSpec((self.hidden,), kind="vector")
        return s

    def bind(self, params, compute_dtype):
        w = torch.cat([params["q_proj.weight"], params["k_proj.weight"], params["v_proj.weight"]], dim=0)
        b = None
        if self.qkv_bias:
            bs = [params["q_proj.bias"], params["k_proj.bias"], params["v_proj.bias"]]
            dt = torch.float32 if any(x.dtype == torch.float32 for x in bs) else bs[0].dtype
            b = torch.cat([x.to(dt) for x in bs]).contiguous()
        self.qkv = Linear(w.contiguous(), b)
        self.o = Linear(params["o_proj.weight"], params.get("o_proj.bias"))
        if self.position is not None:
            self.position.prepare(w.device)

    def cuda_modules(self, compute_dtype):
        mods = ["elementwise", "attention_generic"]
        if compute_dtype == torch.bfloat16:
            mods += ["attention_decode", "attention_prefill", "attention_prefill_tc"]
        return mods

    def cache_request(self):
        return KVRequest(self.n_kv_heads, self.head_dim, self.window)

    # rows of the query tiles of the two tiled prefill kernels (csrc/attention_prefill.cu, attention_prefill_tc.cu)
    TILE_ROWS = {"attention_tiles64": 64, "attention_tiles128": 128}

    def step_table_names(self):
        return tuple(self.TILE_ROWS)

    def step_table(self, name, batch):
        """(sequence, first row) of every query tile of the step's new tokens, sorted by the keys a tile sees (the
        kernels start with the heaviest): decided on the host so that the device never searches.  Steps of one token
        per sequence need none."""
        if batch.is_decode:
            return np.zeros((0,), dtype=np.int32)
        rows = self.TILE_ROWS[name]
        tiles = [(i, q0) for i in range(batch.B) for q0 in range(0, int(batch.n_new[i]), rows)]
        tiles.sort(key=lambda t: int(batch.starts[t[0]]) + t[1])
        return np.asarray(tiles, dtype=np.int32).reshape(-1)

    def forward(self, ctx, y, cache_view, stream):
        q = self.project_into_cache(ctx, y, cache_view)                     # rotated q; k, v are in the cache
        o = self.attend(ctx, q, cache_view)
        self.o.add_to_stream(ctx, o, stream)

    def project_into_cache(self, ctx, y, view):
        """q/k/v projection (+ bias), rotation, cache write; returns rotated q [T, >= heads*head_dim].

        With few tokens on the tensor-core path the product is K-split for parallelism and the
        rotation kernel sums the 32-bit partial sums (and the bias) itself, so q/k/v never
        exist as an intermediate bfloat16 tensor.
        """
        tc = kernels.tensor_core
        w, bias = self.qkv.weight, self.qkv.bias
        y, row_ss = ctx.unpack_rows(y, w, tc.PARTIAL)
        rot = dict((self.position.rotation() if self.position is not None else None) or dict(inv_freq=None, rot_dim=0))
        inv_freq = rot.pop("inv_freq")
        rope = dict(rot_dim=rot["rot_dim"], interleaved=rot.get("interleaved", False), tok_seq=ctx.tok_seq, tok_pos=ctx.tok_pos, seq_slot=ctx.seq_slot,
                    block_table=view.block_table, k_pages=view.k_pages, v_pages=view.v_pages, write_kv=view.writes)
        if y.shape[0] <= tc.SKINNY_MAX_TOKENS and ctx.uses_tensor_cores(y, w, tc.PARTIAL):
            splits = tc.split_k_for(w.shape[0], w.shape[1], tokens=y.shape[0])
            if splits > 1:
                parts = tc.gemm_tc_skinny(y, w, mode=tc.PARTIAL, splits=splits, row_ss=row_ss)
                return kernels.rope_kv_write(parts, self.n_heads, self.n_kv_heads, self.head_dim,
                                             inv_freq, bias=bias, compute_dtype=ctx.compute_dtype,
                                             **rope)
        if row_ss is not None:
            y = ScaledRows(y, row_ss[0], row_ss[1], w.shape[1])
        elif y.shape[0] <= tc.SKINNY_MAX_TOKENS and not ctx.uses_tensor_cores(y, w, tc.STORE):
            splits = kernels.split_k_for_simt(w.shape[0], w.shape[1])
            if splits > 1:                           # CUDA-core product of few tokens: the same scheme
                parts = kernels.gemm_simt(y, w, splits=splits)
                return kernels.rope_kv_write(parts, self.n_heads, self.n_kv_heads, self.head_dim,
                                             inv_freq, bias=bias, compute_dtype=ctx.compute_dtype,
                                             **rope)
        qkv = ctx.matmul(y, w, bias)
        return kernels.rope_kv_write(qkv, self.n_heads, self.n_kv_heads, self.head_dim,
                                     inv_freq, **rope)

    def attend(self, ctx, q, view):
        """Attention of the step's tokens over the cache; q is the first heads*head_dim columns of ``q``."""
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        tiles64, tiles128 = ctx.tables.get("attention_tiles64"), ctx.tables.get("attention_tiles128")
        longest = ctx.model_cache_limit if ctx.replayed else ctx.max_end
        if (ctx.is_decode and ctx.compute_dtype == torch.bfloat16 and ctx.options.tuned_attention
                and kernels.attention_decode_supported(nh, nkv, hd)):
            if ctx.options.clustered_decode:
                # a cluster of 1..8 CTAs per (sequence, kv head), every warp on its own tiles of keys, merged
                # through distributed shared memory: no scratch memory, no second pass, any context length
                return kernels.attention_decode_warps(
                    q, nh, nkv, hd, view.k_pages, view.v_pages, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot,
                    view.block_table, self.scale, view.window,
                    splits=kernels.decode_splits(ctx.B, nkv, longest, view.window))
            if longest <= kernels.DECODE_CHUNK * kernels.DECODE_CHUNK:
                # the earlier kernel: one CTA per 128-key chunk, partial results merged through scratch memory
                need = max(1, (longest + kernels.DECODE_CHUNK - 1) // kernels.DECODE_CHUNK)
                max_chunks = 1
                while max_chunks < need:                   # powers of two: few distinct scratch sizes
                    max_chunks *= 2
                cap = 1
                while cap < ctx.B:
                    cap *= 2
                n_o, n_ml, n_c = kernels.attention_decode_scratch(cap, nh, nkv, hd, max_chunks)
                scratch = ctx.model.scratch
                return kernels.attention_decode(
                    q, nh, nkv, hd, view.k_pages, view.v_pages, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot,
                    view.block_table, self.scale, view.window, max_chunks,
                    scratch("attn_decode_o", n_o, torch.float32), scratch("attn_decode_ml", n_ml, torch.float32),
                    kernels.tensor_core.register_counters(scratch("attn_decode_counters", n_c, torch.int32)))
        if (not ctx.is_decode and ctx.compute_dtype == torch.bfloat16 and ctx.options.tuned_attention
                and ctx.options.tcgen05_attention and tiles128 is not None and tiles128.numel() > 0
                and kernels.attention_prefill_tc_supported(nh, nkv, hd)
                and q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0):
            return kernels.attention_prefill_tc(q, nh, nkv, hd, view.k_pages, view.v_pages, tiles128,
                                                ctx.seq_slot, ctx.seq_start, ctx.seq_nnew, ctx.cu_q,
                                                view.block_table, self.scale, view.window)
        if (not ctx.is_decode and ctx.compute_dtype == torch.bfloat16 and ctx.options.tuned_attention
                and tiles64 is not None and tiles64.numel() > 0 and kernels.attention_prefill_supported(nh, nkv, hd)
                and q.data_ptr() % 4 == 0 and q.stride(0) % 2 == 0):
            return kernels.attention_prefill(q, nh, nkv, hd, view.k_pages, view.v_pages, tiles64, ctx.seq_slot,
                                             ctx.seq_start, ctx.seq_nnew, ctx.cu_q, view.block_table, self.scale,
                                             view.window)
        return kernels.attention_generic(q, nh, nkv, hd, view.k_pages, view.v_pages, ctx.tok_seq, ctx.tok_pos,
                                         ctx.seq_slot, view.block_table, self.scale, view.window)

