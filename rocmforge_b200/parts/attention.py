"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import kernels
from ..cache.requests import KVRequest
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

    def forward(self, ctx, y, cache_view, stream):
        q = ctx.project_qkv_into_cache(y, self, cache_view)                 # rotated q; k, v are in the cache
        o = ctx.attention(q, self, cache_view)
        self.o.add_to_stream(ctx, o, stream)
