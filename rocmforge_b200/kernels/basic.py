"""Python faces of the plain kernels: embedding, add+RMSNorm, rotation + cache write,
SwiGLU, the CUDA-core matrix product, the generic attention and argmax.

Each function checks shapes and dtypes, then launches on torch's current stream.
"""
from __future__ import annotations

import functools

import torch

from ._ffi import (KernelError, sm_count as device_sm_count, c_float, c_int, c_ll, c_void_p, check, dtype_code, fn, need, need_cuda,
                   ptr, stream)

PAGE = 64      # tokens per cache page (RF_PAGE in csrc/common.cuh)


@functools.lru_cache(None)
def _f(module, name, *argtypes):
    return fn(module, name, list(argtypes))


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[ids[t]] widened to float32."""
    need_cuda(table, ids)
    need(table.dim() == 2 and table.is_contiguous(), "embed: table must be a contiguous matrix")
    need(ids.dtype == torch.int32 and ids.dim() == 1, "embed: ids must be a 1-d int32 tensor")
    V, H = table.shape
    T = ids.shape[0]
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    f = _f("elementwise", "rf_embed", c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p)
    check(f(dtype_code(table.dtype), ptr(table), ptr(ids), ptr(out), T, H, V, stream()), "embed")
    return out


def add_rmsnorm(h: torch.Tensor, weight: torch.Tensor, eps: float, compute_dtype: torch.dtype,
                pending: torch.Tensor | None = None, rows: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """y = rmsnorm(h + pending) * weight.

    ``h`` [T, H] float32 is the residual stream.  ``pending`` is None, a float32
    [S, T, H] stack of partial sums, or a [T, H] tensor of the compute dtype; without
    ``rows`` it is added into ``h`` in place.  With ``rows`` (int32 indices) only those
    rows are normalised and ``h`` is left untouched.
    """
    need_cuda(h, weight, pending, rows)
    need(h.dtype == torch.float32 and h.dim() == 2 and h.is_contiguous(), "add_rmsnorm: h must be [T,H] float32")
    T, H = h.shape
    need(weight.shape == (H,) and weight.dtype in (torch.float32, torch.bfloat16),
         "add_rmsnorm: weight must be [H] in float32 or bfloat16")
    kind, n_pending, pstride = 0, 0, 0
    if pending is not None:
        need(pending.is_contiguous(), "add_rmsnorm: pending must be contiguous")
        if pending.dtype == torch.float32 and pending.dim() == 3 and pending.shape[1:] == (T, H):
            kind, n_pending, pstride = 1, pending.shape[0], T * H
        elif pending.dtype == torch.float32 and pending.shape == (T, H) and compute_dtype == torch.float32:
            kind = 2
        elif pending.dtype == torch.float32 and pending.shape == (T, H):
            kind, n_pending, pstride = 1, 1, T * H
        elif pending.dtype == compute_dtype and pending.shape == (T, H):
            kind = 2
        else:
            raise KernelError(f"add_rmsnorm: pending of shape {tuple(pending.shape)} / {pending.dtype} "
                              f"does not fit h {tuple(h.shape)}")
    n_rows = T
    if rows is not None:
        need(rows.dtype == torch.int32 and rows.dim() == 1, "add_rmsnorm: rows must be 1-d int32")
        n_rows = rows.shape[0]
    if out is None:
        out = torch.empty((n_rows, H), dtype=compute_dtype, device=h.device)
    from .tensor_core import status_word
    f = _f("elementwise", "rf_add_rmsnorm", c_int, c_void_p, c_void_p, c_int, c_int, c_ll, c_void_p, c_int,
           c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p)
    check(f(dtype_code(compute_dtype), ptr(h), ptr(pending), kind, n_pending, pstride, ptr(weight),
            int(weight.dtype == torch.float32), float(eps), ptr(out), ptr(rows), n_rows, H,
            ptr(status_word(h.device)), stream()),
          f"add_rmsnorm (H={H})")
    return out


def rope_kv_write(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, inv_freq: torch.Tensor,
                  tok_seq, tok_pos, seq_slot, block_table: torch.Tensor,
                  k_pages: torch.Tensor | None, v_pages: torch.Tensor | None, write_kv: bool = True, *,
                  bias: torch.Tensor | None = None, compute_dtype: torch.dtype | None = None,
                  q_out: torch.Tensor | None = None, rot_dim: int | None = None,
                  interleaved: bool = False) -> torch.Tensor:
    """Rotate q and k by position; write rotated k and v into their cache pages; return q.

    The first ``rot_dim`` elements of every query and key head turn (default: the whole head; 0: none, and
    ``inv_freq`` may then be None), as pairs (i, i + rot_dim/2) or, ``interleaved``, (2i, 2i+1), pair i by the angle
    position * inv_freq[i]; the other elements pass through.

    ``qkv`` is [T, (heads + 2 kv_heads) * head_dim] in the compute dtype (q is then rotated in place and
    the returned q is a view of it), or a float32 stack [S, T, ...] of partial sums of a K-split product,
    to which ``bias`` is added (q then goes to a new [T, heads * head_dim] tensor of ``compute_dtype``).
    """
    need_cuda(qkv, inv_freq, tok_seq, tok_pos, seq_slot, block_table, k_pages, v_pages, bias)
    width = (n_heads + 2 * n_kv_heads) * head_dim
    partials = qkv.dim() == 3
    if partials:
        need(qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.shape[2] == width,
             "rope_kv_write: partial sums must be a contiguous float32 [S, T, width] stack")
        need(compute_dtype is not None, "rope_kv_write: partial sums need the compute dtype")
        S, T = qkv.shape[0], qkv.shape[1]
        dt = compute_dtype
        if q_out is None:
            q_out = torch.empty((T, n_heads * head_dim), dtype=dt, device=qkv.device)
        row_stride, pstride = width, T * width
    else:
        need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] == width,
             "rope_kv_write: qkv must be [T, (heads + 2 kv_heads) * head_dim]")
        need(bias is None, "rope_kv_write: a bias goes with partial sums only")
        S, T, dt = 0, qkv.shape[0], qkv.dtype
        q_out = qkv
        row_stride, pstride = qkv.stride(0), 0
    rot_dim = head_dim if rot_dim is None else int(rot_dim)
    need(0 <= rot_dim <= head_dim and rot_dim % 2 == 0, f"rope_kv_write: rot_dim {rot_dim} must be even and at most head_dim")
    need(rot_dim == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2),
         "rope_kv_write: inv_freq must hold rot_dim/2 float32 frequencies")
    if write_kv:
        for p in (k_pages, v_pages):
            need(p is not None and p.dtype == dt and p.is_contiguous()
                 and tuple(p.shape[1:]) == (n_kv_heads, PAGE, head_dim),
                 "rope_kv_write: pages must be [n_pages, kv_heads, 64, head_dim] of the compute dtype")
    f = _f("elementwise", "rf_rope_kv_write", c_int, c_void_p, c_int, c_int, c_ll, c_void_p, c_int, c_void_p, c_int,
           c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
           c_int, c_int, c_int, c_void_p)
    check(f(dtype_code(dt), ptr(qkv), row_stride, S, pstride, ptr(bias),
            int(bias is not None and bias.dtype == torch.float32), ptr(q_out), q_out.stride(0), n_heads, n_kv_heads,
            head_dim, ptr(inv_freq), ptr(tok_seq), ptr(tok_pos), ptr(seq_slot), ptr(block_table),
            block_table.shape[1], ptr(k_pages), ptr(v_pages), int(write_kv), T, rot_dim, int(interleaved), stream()),
          "rope_kv_write")
    return q_out


def swiglu(gu: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """a[t, j] = silu(gu[t, 2j]) * gu[t, 2j+1]."""
    need_cuda(gu)
    need(gu.dim() == 2 and gu.is_contiguous() and gu.shape[1] % 2 == 0, "swiglu: input must be [T, 2I]")
    T, I2 = gu.shape
    if out is None:
        out = torch.empty((T, I2 // 2), dtype=gu.dtype, device=gu.device)
    f = _f("elementwise", "rf_swiglu", c_int, c_void_p, c_void_p, c_int, c_int, c_void_p)
    check(f(dtype_code(gu.dtype), ptr(gu), ptr(out), T, I2 // 2, stream()), "swiglu")
    return out


def split_k_for_simt(N: int, K: int, sm_count: int | None = None) -> int:
    """K splits of a CUDA-core product of few tokens, from N and K alone (never from the batch): about two CTAs
    per SM, every split at least 4 blocks of 16."""
    sm_count = sm_count or device_sm_count()
    tiles = (N + 127) // 128
    kb = (K + 15) // 16
    if tiles >= 2 * sm_count or kb < 8:
        return 1
    splits = max(1, min((2 * sm_count) // tiles, kb // 4))
    per = (kb + splits - 1) // splits
    return (kb + per - 1) // per                   # no empty split


def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *,
              out: torch.Tensor | None = None, out_f32: bool = False, accumulate: bool = False,
              splits: int = 0) -> torch.Tensor:
    """y = x @ w.T (+ bias) on CUDA cores with 32-bit sums.

    out_f32: the result is float32 whatever the inputs; accumulate: added into ``out`` (float32);
    splits >= 1: the result is the float32 stack [splits, M, N] of partial sums over K ranges (no bias).
    """
    need_cuda(x, w, bias, out)
    need(x.dim() == 2 and w.dim() == 2 and x.dtype == w.dtype and x.stride(1) == 1 and w.is_contiguous(),
         "gemm: x [M,K] and w [N,K] must share a dtype and be row-major")
    M, K = x.shape
    N = w.shape[0]
    need(w.shape[1] == K, f"gemm: inner sizes differ ({K} vs {w.shape[1]})")
    if bias is not None:
        need(bias.shape == (N,) and bias.dtype in (torch.float32, torch.bfloat16), "gemm: bias must be [N]")
    f = _f("gemm_simt", "rf_gemm_simt", c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
           c_int, c_int, c_int, c_int, c_int, c_void_p)
    if splits >= 1:
        need(not accumulate and out is None and bias is None, "gemm: partial sums take no bias and no output tensor")
        out = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
        check(f(dtype_code(x.dtype), ptr(x), ptr(w), ptr(None), 0, ptr(out), M, N, K, x.stride(0), N, 3, splits, stream()),
              f"gemm_simt ({M}x{N}x{K}, {splits} partial sums)")
        return out
    mode = 2 if accumulate else (1 if out_f32 else 0)
    odt = torch.float32 if mode else x.dtype
    if out is None:
        need(not accumulate, "gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=odt, device=x.device)
    need(out.shape == (M, N) and out.dtype == odt and out.stride(1) == 1, "gemm: output has the wrong shape or dtype")
    check(f(dtype_code(x.dtype), ptr(x), ptr(w), ptr(bias), int(bias is not None and bias.dtype == torch.float32),
            ptr(out), M, N, K, x.stride(0), out.stride(0), mode, 1, stream()), f"gemm_simt ({M}x{N}x{K})")
    return out


def attention_generic(q: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, k_pages, v_pages,
                      tok_seq, tok_pos, seq_slot, block_table, scale: float, window: int | None,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of the T new tokens over the paged cache (their own keys included)."""
    need_cuda(q, k_pages, v_pages, tok_seq, tok_pos, seq_slot, block_table)
    T = q.shape[0]
    need(q.dim() == 2 and q.stride(1) == 1, "attention: q must be [T, >= heads*head_dim] with unit inner stride")
    need(k_pages.dtype == q.dtype and v_pages.dtype == q.dtype, "attention: cache dtype differs from q")
    need(tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim) and k_pages.is_contiguous()
         and v_pages.shape == k_pages.shape and v_pages.is_contiguous(), "attention: bad cache page shape")
    if out is None:
        out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    f = _f("attention_generic", "rf_attention_generic", c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
           c_void_p)
    check(f(dtype_code(q.dtype), ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages),
            ptr(tok_seq), ptr(tok_pos), ptr(seq_slot), ptr(block_table), block_table.shape[1], n_heads,
            n_kv_heads, head_dim, float(scale), int(window or 0), T, stream()),
          f"attention_generic (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim})")
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Row-wise argmax of float32 logits; of equal maxima the highest index."""
    need_cuda(logits)
    need(logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1,
         "argmax: logits must be [rows, vocab] float32")
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    f = _f("sampling", "rf_argmax", c_void_p, c_int, c_int, c_ll, c_void_p, c_void_p)
    check(f(ptr(logits), R, V, logits.stride(0), ptr(out), stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: float, top_p: float, top_k: int, seeds: torch.Tensor,
           draw_counter: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """One seeded draw per row after temperature, top-k and nucleus filtering.

    ``seeds`` [rows] int64 holds each row's 64-bit LCG seed; ``draw_counter`` (a device int32
    scalar) is added to every seed, so that a replayed step can advance its draws without the host.
    """
    need_cuda(logits, seeds, draw_counter)
    need(logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1,
         "sample: logits must be [rows, vocab] float32")
    R, V = logits.shape
    need(seeds.dtype == torch.int64 and seeds.shape == (R,), "sample: seeds must be [rows] int64")
    need(temperature > 0.0, "sample: temperature must be positive (0 means argmax)")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    f = _f("sampling", "rf_sample", c_void_p, c_int, c_int, c_ll, c_float, c_float, c_int, c_void_p, c_void_p,
           c_void_p, c_void_p)
    check(f(ptr(logits), R, V, logits.stride(0), float(temperature), float(top_p), int(top_k), ptr(seeds),
            ptr(draw_counter), ptr(out), stream()), "sample")
    return out


def set_sample_cached(on: bool) -> None:
    """Which sampler ``sample`` launches where both can run: the one that keeps a CTA's slice of the row in shared
    memory (the default), or the one that walks the row in global memory (it also serves vocabularies whose slices do
    not fit).  Both give the same token."""
    check(_f("sampling", "rf_sample_set_cached", c_int)(1 if on else 0), "set_sample_cached")


def advance_decode(tokens, tok_pos, seq_start, sampled) -> None:
    """tokens <- sampled; positions and starts += 1 (one token per sequence), all on the device."""
    need_cuda(tokens, tok_pos, seq_start, sampled)
    B = tokens.shape[0]
    need(all(t.dtype == torch.int32 and t.shape == (B,) for t in (tokens, tok_pos, seq_start, sampled)),
         "advance_decode: four int32 arrays of one length")
    f = _f("sampling", "rf_advance_decode", c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p)
    check(f(ptr(tokens), ptr(tok_pos), ptr(seq_start), ptr(sampled), B, stream()), "advance_decode")


def gather_tokens(tokens, ids, row_map) -> None:
    """tokens[i] = ids[row_map[i]] on the device (all int32)."""
    need_cuda(tokens, ids, row_map)
    B = tokens.shape[0]
    need(all(t.dtype == torch.int32 and t.dim() == 1 for t in (tokens, ids, row_map)) and row_map.shape[0] == B,
         "gather_tokens: int32 vectors, one map entry per token")
    f = _f("sampling", "rf_gather_tokens", c_void_p, c_void_p, c_void_p, c_int, c_void_p)
    check(f(ptr(tokens), ptr(ids), ptr(row_map), B, stream()), "gather_tokens")


def attention_decode_supported(n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    f = _f("attention_decode", "rf_attention_decode_supported", c_int, c_int, c_int)
    return bool(f(n_heads, n_kv_heads, head_dim))


DECODE_CHUNK = 128


def attention_decode_scratch(B: int, n_heads: int, n_kv_heads: int, head_dim: int, max_chunks: int):
    """Element counts (partial outputs, partial max/sum, counters) the decode attention needs for B sequences."""
    return (B * n_heads * max_chunks * head_dim, B * n_heads * max_chunks * 2, B * n_kv_heads)


def attention_decode(q: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, k_pages, v_pages,
                     tok_seq, tok_pos, seq_slot, block_table, scale: float, window: int | None, max_chunks: int,
                     part_o: torch.Tensor, part_ml: torch.Tensor, counters: torch.Tensor,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """One new token per sequence over the bfloat16 paged cache, keys in chunks of 128.

    ``max_chunks`` must cover the longest sequence (ceil(length / 128)); ``part_o``, ``part_ml`` (float32)
    and ``counters`` (int32, zero before the first call; the kernel leaves them zero) are scratch of at
    least ``attention_decode_scratch`` elements.
    """
    need_cuda(q, k_pages, v_pages, tok_seq, tok_pos, seq_slot, block_table, part_o, part_ml, counters)
    B = q.shape[0]
    need(q.dtype == torch.bfloat16 and q.dim() == 2 and q.stride(1) == 1, "attention_decode: q must be bfloat16 [B, ...]")
    need(k_pages.dtype == torch.bfloat16 and tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim)
         and k_pages.is_contiguous() and v_pages.shape == k_pages.shape and v_pages.is_contiguous(),
         "attention_decode: bad cache page shape or dtype")
    need(attention_decode_supported(n_heads, n_kv_heads, head_dim),
         f"attention_decode: heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim} is not supported")
    n_o, n_ml, n_c = attention_decode_scratch(B, n_heads, n_kv_heads, head_dim, max_chunks)
    need(part_o.dtype == torch.float32 and part_o.numel() >= n_o and part_ml.dtype == torch.float32
         and part_ml.numel() >= n_ml and counters.dtype == torch.int32 and counters.numel() >= n_c,
         "attention_decode: scratch tensors are too small")
    need(q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0, "attention_decode: q rows must be 16-byte aligned")
    if out is None:
        out = torch.empty((B, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    f = _f("attention_decode", "rf_attention_decode", c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
           c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p,
           c_void_p, c_void_p, c_void_p)
    from .tensor_core import status_word
    check(f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages), ptr(tok_seq), ptr(tok_pos),
            ptr(seq_slot), ptr(block_table), block_table.shape[1], n_heads, n_kv_heads, head_dim, float(scale),
            int(window or 0), B, max_chunks, ptr(part_o), ptr(part_ml), ptr(counters), ptr(status_word(q.device)),
            stream()),
          f"attention_decode (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim})")
    return out


PREFILL_TILE = 64


def attention_prefill_supported(n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    f = _f("attention_prefill", "rf_attention_prefill_supported", c_int, c_int, c_int)
    return bool(f(n_heads, n_kv_heads, head_dim))


def attention_prefill(q: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, k_pages, v_pages,
                      q_tiles: torch.Tensor, seq_slot, seq_start, seq_nnew, cu_q, block_table, scale: float,
                      window: int | None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Tiled causal attention of the new tokens over the bfloat16 paged cache (head_dim 64 or 128).

    ``q_tiles`` is an int32 array of (sequence index, first row within the sequence's new tokens) pairs,
    one per 64-row tile, built on the host.
    """
    need_cuda(q, k_pages, v_pages, q_tiles, seq_slot, seq_start, seq_nnew, cu_q, block_table)
    T = q.shape[0]
    need(q.dtype == torch.bfloat16 and q.dim() == 2 and q.stride(1) == 1, "attention_prefill: q must be bfloat16 [T, ...]")
    need(k_pages.dtype == torch.bfloat16 and tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim)
         and k_pages.is_contiguous() and v_pages.shape == k_pages.shape and v_pages.is_contiguous(),
         "attention_prefill: bad cache page shape or dtype")
    need(attention_prefill_supported(n_heads, n_kv_heads, head_dim),
         f"attention_prefill: heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim} is not supported")
    need(q_tiles.dtype == torch.int32 and q_tiles.numel() % 2 == 0, "attention_prefill: q_tiles must be int32 pairs")
    if out is None:
        out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    from .tensor_core import status_word
    f = _f("attention_prefill", "rf_attention_prefill", c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_ll,
           c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int,
           c_void_p, c_void_p)
    check(f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages), k_pages.shape[0], ptr(q_tiles),
            q_tiles.numel() // 2, ptr(seq_slot), ptr(seq_start), ptr(seq_nnew), ptr(cu_q), ptr(block_table),
            block_table.shape[1], n_heads, n_kv_heads, head_dim, float(scale), int(window or 0),
            ptr(status_word(q.device)), stream()),
          f"attention_prefill (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim})")
    return out


def decode_splits(B: int, n_kv_heads: int, longest: int | None = None, window: int | None = None) -> int:
    """CTAs that share one (sequence, kv head) in the clustered decode attention, from the batch and the
    longest context the launch may meet (a captured graph keeps its launch shape): about one CTA per SM,
    at most one CTA per page, and clusters of 8 only for very small batches, where nothing else fills the
    GPU.  Measured at 28 layers, 4 kv heads of 7 query heads, ms per decode step: batch 1 / 3,800 keys:
    1, 2, 4, 8 CTAs 3.45, 3.16, 2.92, 2.85; batch 8 / 1,900 keys: 3.21, 3.10, 3.01, 3.05; batch 32 / 512:
    3.54, 3.54, 3.72; batch 64 / 512: 3.76, 4.04."""
    pairs = max(1, B * n_kv_heads)
    s = 1
    while s < 8 and pairs * s * 2 <= device_sm_count() * 7 // 8:          # 128 on the 148 SMs these numbers were taken on
        s *= 2
    if s == 8 and pairs > 8:
        s = 4
    if longest is not None:
        pages = decode_pages(longest, window)
        # one sequence with a long context: clusters of 16 (beyond the portable size; four of them still find a
        # GPC each).  28 heads on 4 kv heads, 16,000 keys: 17.7 -> 11.8 us a layer; 8 such clusters were slower
        if s == 8 and pairs <= 4 and pages >= 32:
            s = 16
        while s > 1 and s > pages:
            s //= 2
    return s


def decode_pages(longest: int, window: int | None) -> int:
    """Most pages of 64 positions that a new token at context length ``longest`` reads."""
    pages = (max(1, longest) + PAGE - 1) // PAGE
    if window:
        pages = min(pages, (window + PAGE - 2) // PAGE + 1)
    return pages


def attention_decode_warps(q: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, k_pages, v_pages,
                           tok_seq, tok_pos, seq_slot, block_table, scale: float, window: int | None,
                           splits: int | None = None, warps: int | None = None,
                           out: torch.Tensor | None = None) -> torch.Tensor:
    """One new token per sequence over the bfloat16 paged cache: a cluster of ``splits`` CTAs per (sequence,
    kv head), every warp on its own tiles of keys; merged through distributed shared memory.  ``warps``
    per CTA: 8 while one CTA per SM is enough for the batch, else 4 (three CTAs fit an SM)."""
    need_cuda(q, k_pages, v_pages, tok_seq, tok_pos, seq_slot, block_table)
    B = q.shape[0]
    need(q.dtype == torch.bfloat16 and q.dim() == 2 and q.stride(1) == 1, "attention_decode: q must be bfloat16 [B, ...]")
    need(k_pages.dtype == torch.bfloat16 and tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim)
         and k_pages.is_contiguous() and v_pages.shape == k_pages.shape and v_pages.is_contiguous(),
         "attention_decode: bad cache page shape or dtype")
    need(attention_decode_supported(n_heads, n_kv_heads, head_dim),
         f"attention_decode: heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim} is not supported")
    need(q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0, "attention_decode: q rows must be 16-byte aligned")
    if splits is None:
        splits = decode_splits(B, n_kv_heads)
    if warps is None:
        warps = 8 if B * n_kv_heads * splits <= device_sm_count(q.device) else 4
    if out is None:
        out = torch.empty((B, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    from .tensor_core import status_word
    f = _f("attention_decode", "rf_attention_decode_warps", c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
           c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int,
           c_void_p, c_void_p)
    check(f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages), k_pages.shape[0], ptr(tok_seq),
            ptr(tok_pos), ptr(seq_slot), ptr(block_table), block_table.shape[1], n_heads, n_kv_heads, head_dim,
            float(scale), int(window or 0), B, splits, warps, ptr(status_word(q.device)), stream()),
          f"attention_decode_warps (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim}, splits={splits})")
    return out


PREFILL_TC_TILE = 128


def attention_prefill_tc_supported(n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    f = _f("attention_prefill_tc", "rf_attention_prefill_tc_supported", c_int, c_int, c_int)
    return bool(f(n_heads, n_kv_heads, head_dim))


def attention_prefill_tc(q: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, k_pages, v_pages,
                         q_tiles: torch.Tensor, seq_slot, seq_start, seq_nnew, cu_q, block_table, scale: float,
                         window: int | None, out: torch.Tensor | None = None) -> torch.Tensor:
    """The same attention as ``attention_prefill`` with both products as tcgen05.mma (accumulators in tensor
    memory); ``q_tiles`` holds (sequence, first row) pairs of 128-row tiles."""
    need_cuda(q, k_pages, v_pages, q_tiles, seq_slot, seq_start, seq_nnew, cu_q, block_table)
    T = q.shape[0]
    need(q.dtype == torch.bfloat16 and q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= n_heads * head_dim,
         "attention_prefill_tc: q must be bfloat16 [T, >= heads*head_dim]")
    need(q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0, "attention_prefill_tc: q rows must be 16-byte aligned")
    need(k_pages.dtype == torch.bfloat16 and tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim)
         and k_pages.is_contiguous() and v_pages.shape == k_pages.shape and v_pages.is_contiguous(),
         "attention_prefill_tc: bad cache page shape or dtype")
    need(attention_prefill_tc_supported(n_heads, n_kv_heads, head_dim),
         f"attention_prefill_tc: heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim} is not supported")
    need(q_tiles.dtype == torch.int32 and q_tiles.numel() % 2 == 0, "attention_prefill_tc: q_tiles must be int32 pairs")
    if out is None:
        out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    from .tensor_core import status_word
    f = _f("attention_prefill_tc", "rf_attention_prefill_tc", c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
           c_ll, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
           c_int, c_void_p, c_void_p)
    check(f(ptr(q), q.stride(0), T, ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages), k_pages.shape[0], ptr(q_tiles),
            q_tiles.numel() // 2, ptr(seq_slot), ptr(seq_start), ptr(seq_nnew), ptr(cu_q), ptr(block_table),
            block_table.shape[1], n_heads, n_kv_heads, head_dim, float(scale), int(window or 0),
            ptr(status_word(q.device)), stream()),
          f"attention_prefill_tc (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim})")
    return out
