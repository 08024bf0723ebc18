"""Plain, slow implementation of the Qwen2.5 dense decoder, used as the test oracle.

It rests on the formulas of maeddesg/ROCmForge's CPU backend (Rust), which can be
neither imported nor compiled where these tests run (no Rust toolchain, GGUF-only
loader), so every function below cites the file and lines of the reference that it
restates.  It shares no code with ``rocmforge_b200``: it reads the model folder
with the ``safetensors`` package, keeps no cache, and always runs whole sequences.

All arithmetic is done in ``dtype`` (float64 by default, so that the oracle's own
rounding is far below every tolerance used against it), except the rotation angle,
which the reference computes in 32-bit (``pos as f32 * freq``): the angle is
rounded to float32 first, then its sine and cosine are taken exactly.
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------- folder

def read_folder(folder: str):
    """Return (config dict, {tensor name: torch tensor}) of a model folder."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    return cfg, tensors


def head_dim_of(cfg) -> int:
    # src/loader/metadata.rs:130-143 — explicit head_dim key, else hidden / heads
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


def layer_window(cfg, layer: int):
    """Window (number of keys a query sees, itself included) of a layer, or None.

    The reference has no window; the meaning of the three config.json keys is the
    architecture's own: with ``use_sliding_window`` the layers with index >=
    ``max_window_layers`` attend to the last ``sliding_window`` positions only.
    """
    if not cfg.get("use_sliding_window", False):
        return None
    w = cfg.get("sliding_window")
    if w is None:
        return None
    if layer >= int(cfg.get("max_window_layers", 0)):
        return int(w)
    return None


# --------------------------------------------------------------------------- parts

def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """x = E[token], a plain row gather without scaling (src/cpu/quant.rs:114-119,
    src/gpu/forward.rs:826-883)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """out[i] = x[i] / sqrt(sum(x^2)/n + eps) * w[i]  (src/cpu/ops.rs:32-46,
    hip_kernels/norm.hip:68,82)."""
    n = x.shape[-1]
    sum_sq = (x * x).sum(dim=-1, keepdim=True)
    rms = torch.sqrt(sum_sq / n + eps)
    return x / rms * w


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """Y[s,o] = dot(W[o,:], X[s,:]) (src/cpu/ops.rs:342-352); the bias is added
    after the product (src/cpu/ops.rs:308-323, src/gpu/forward.rs:974-1000)."""
    y = x @ w.t()
    if b is not None:
        y = y + b
    return y


def rope_neox(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Split-half rotation over the whole head (src/cpu/ops.rs:69-98 with neox=true,
    hip_kernels/rope.hip:57-90).

    x: [T, heads, head_dim]; positions: [T].  freq_i = 1/theta^(2i/d);
    angle = pos * freq_i in 32-bit; pairs are (i, i + d/2).
    """
    T, nh, hd = x.shape
    half = hd // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = (1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2.0 * i / hd)).to(torch.float32)
    angle32 = positions.to(torch.float32)[:, None] * freq.to(positions.device)[None, :]      # 32-bit product
    angle = angle32.to(torch.float64)
    cos = torch.cos(angle).to(x.dtype)[:, None, :]
    sin = torch.sin(angle).to(x.dtype)[:, None, :]
    x0 = x[..., :half]
    x1 = x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)


def causal_attention(q, k, v, window=None):
    """Causal grouped-query attention of one whole sequence (src/cpu/ops.rs:253-303).

    q: [T, nh, hd], k/v: [T, nkv, hd].  Head h reads kv head h // (nh/nkv); the score
    is dot(q,k)/sqrt(hd); position s sees 0..=s (src/cpu/ops.rs:282), narrowed to
    the last ``window`` positions when a window is given; the softmax is the
    max-subtracted exponential sum (src/cpu/ops.rs:164-182).
    """
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    pos = torch.arange(T, device=q.device)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed = allowed & (pos[None, :] > pos[:, None] - window)
    for h in range(nh):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].t()) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        w = torch.exp(s - m)
        out[:, h, :] = (w @ v[:, kh, :]) / w.sum(dim=-1, keepdim=True)
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x))  (src/cpu/ops.rs:119-123)."""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(y, w_gate, w_up, w_down):
    """down(silu(gate(y)) * up(y)), no biases (src/cpu/ops.rs:125-131,
    src/gpu/forward.rs:1094-1161)."""
    return linear(silu(linear(y, w_gate)) * linear(y, w_up), w_down)


def attention_block(y, positions, p, prefix, cfg, layer):
    """q/k/v projections with bias, rotation of q and k, attention, output
    projection without bias (src/gpu/forward.rs:940-1079)."""
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    hd = head_dim_of(cfg)
    T = y.shape[0]
    q = linear(y, p[prefix + "q_proj.weight"], p.get(prefix + "q_proj.bias")).view(T, nh, hd)
    k = linear(y, p[prefix + "k_proj.weight"], p.get(prefix + "k_proj.bias")).view(T, nkv, hd)
    v = linear(y, p[prefix + "v_proj.weight"], p.get(prefix + "v_proj.bias")).view(T, nkv, hd)
    q = rope_neox(q, positions, cfg["rope_theta"])
    k = rope_neox(k, positions, cfg["rope_theta"])
    o = causal_attention(q, k, v, window=layer_window(cfg, layer))
    return linear(o.reshape(T, nh * hd), p[prefix + "o_proj.weight"])


def decoder_layer(x, positions, p, cfg, layer):
    """Pre-norm block: x += attn(norm(x)); x += mlp(norm(x))
    (src/gpu/forward.rs:886-1195, src/cpu/forward.rs:18-337)."""
    pre = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    y = rms_norm(x, p[pre + "input_layernorm.weight"], eps)
    x = x + attention_block(y, positions, p, pre + "self_attn.", cfg, layer)
    y = rms_norm(x, p[pre + "post_attention_layernorm.weight"], eps)
    x = x + swiglu_mlp(y, p[pre + "mlp.gate_proj.weight"], p[pre + "mlp.up_proj.weight"],
                       p[pre + "mlp.down_proj.weight"])
    return x


class _AsStored(dict):
    """Tensors kept as the file stores them and widened one at a time when a function asks for one:
    a model of real layer widths in float64 all at once would not fit the host's memory."""

    def __init__(self, tensors, dtype):
        super().__init__(tensors)
        self.dtype = dtype

    def __getitem__(self, name):
        return super().__getitem__(name).to(self.dtype)

    def get(self, name, default=None):
        return self[name] if name in self else default

    def stored(self, name):
        return super().__getitem__(name)


def forward_logits(cfg, tensors, token_ids, dtype=torch.float64, rows=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence, no cache
    (src/gpu/forward.rs:1198-1393; the reference keeps the last row only).  ``rows``: only these
    positions go through the final norm and the output matrix (the reference's last-row case, for any rows)."""
    p = tensors if isinstance(tensors, _AsStored) else {k: v.to(dtype) for k, v in tensors.items()}
    device = next(iter(dict.values(p))).device
    ids = torch.as_tensor(token_ids, dtype=torch.long).to(device)
    positions = torch.arange(len(ids), device=device)
    table = p.stored("model.embed_tokens.weight") if isinstance(p, _AsStored) else p["model.embed_tokens.weight"]
    x = embedding(table, ids).to(dtype)          # a row gather: widening the gathered rows is widening the table
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, positions, p, cfg, layer)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long).to(device)]
    x = rms_norm(x, p["model.norm.weight"], cfg["rms_norm_eps"])
    # src/gpu/weights.rs:868-886 — no output matrix means the embedding serves as one
    head = p["lm_head.weight"] if "lm_head.weight" in p else p["model.embed_tokens.weight"]
    return linear(x, head)


class PlainModel:
    """Convenience holder: folder -> logits of whole sequences."""

    def __init__(self, folder: str, dtype=torch.float64, as_stored: bool = False, device="cpu"):
        """``as_stored``: keep the tensors as the file has them and widen each when it is used; ``device``: where
        this plain arithmetic runs (the formulas are the same; models of real layer widths take minutes on a CPU)."""
        self.cfg, tensors = read_folder(folder)
        self.dtype = dtype
        tensors = {k: v.to(device) for k, v in tensors.items()}
        self.tensors = _AsStored(tensors, dtype) if as_stored else {k: v.to(dtype) for k, v in tensors.items()}

    def logits(self, token_ids, rows=None) -> torch.Tensor:
        return forward_logits(self.cfg, self.tensors, token_ids, self.dtype, rows).cpu()
