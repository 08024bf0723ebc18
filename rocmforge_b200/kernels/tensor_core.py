"""Python face of the tcgen05 matrix products (bfloat16 in, 32-bit accumulate)."""
from __future__ import annotations

import functools
from typing import Optional

import torch

from ._ffi import KernelError, sm_count as device_sm_count, c_float, c_int, c_ll, c_void_p, check, fn, need, need_cuda, ptr, stream

STORE, F32, RESIDUAL, SWIGLU, PARTIAL, RESNORM = 0, 1, 2, 3, 4, 5
SKINNY_MAX_TOKENS = 128     # above it the large-M kernels stream the weights better (7B shape, decode step: 128 tokens
                            # 5.09 ms skinny / 6.38 ms clustered; 192 tokens as tiles of 64: 7.78 / 6.73)

_status = {}


def status_word(device) -> torch.Tensor:
    """Device word that a kernel sets when one of its bounded waits runs out."""
    word = _status.get(device)                       # asked at every launch: no string is built on this path
    if word is None:
        key = str(torch.device(device))
        word = _status.get(key)
        if word is None:
            word = _status[key] = torch.zeros((1,), dtype=torch.int32, device=device)
        _status[device] = word
    return word


_counters = {}


def register_counters(t: torch.Tensor) -> torch.Tensor:
    """Arrival counters that kernels leave at zero when they finish; a kernel that gave up may not have, so
    ``check_status`` clears every registered buffer when it finds the status word set."""
    _counters[t.data_ptr()] = t
    return t


def check_status(device) -> None:
    """Raise if a kernel gave up since the last check (synchronises): a bounded wait ran out (a copy or an MMA
    never completed), or a launch did not cover a sequence's length."""
    key = str(torch.device(device))
    if key in _status and int(_status[key].item()) != 0:
        code = int(_status[key].item())
        _status[key].zero_()
        for flags in list(_part_flags.values()) + list(_counters.values()):
            flags.zero_()                          # what the kernel that gave up may have left behind
        raise KernelError(f"a kernel gave up (status {code}: a wait ran out of its limit, or a launch did not cover "
                          "a sequence's length); its results are invalid")


@functools.lru_cache(None)
def _f(name, *argtypes):
    return fn("gemm_tcgen05", name, list(argtypes))


@functools.lru_cache(None)
def supported(M: int, N: int, K: int, mode: int = STORE) -> bool:
    f = _f("rf_gemm_tc_supported", c_int, c_int, c_int, c_int)
    return bool(f(M, N, K, mode))


def _common(x, w, bias, out):
    need_cuda(x, w, bias, out)
    need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "tensor-core gemm: x and w must be bfloat16")
    need(x.dim() == 2 and w.dim() == 2 and x.stride(1) == 1 and w.is_contiguous() and x.shape[1] == w.shape[1],
         "tensor-core gemm: x [M,K] and w [N,K] must be row-major with equal K")
    need(x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and (x.stride(0) * 2) % 16 == 0,
         "tensor-core gemm: operands must be 16-byte aligned")
    if bias is not None:
        need(bias.shape == (w.shape[0],) and bias.dtype in (torch.float32, torch.bfloat16), "gemm: bias must be [N]")


_cluster_ok = None


def cluster_available() -> bool:
    """The clustered kernel lives in an optional module (its cluster-wide tile loads are kept out of runs on several GPUs)."""
    global _cluster_ok
    if _cluster_ok is None:
        from ..csrc import build
        _cluster_ok = build.available("gemm_tcgen05_cluster")
    return _cluster_ok


@functools.lru_cache(None)
def cluster_supported(M: int, N: int, K: int, mode: int = STORE) -> bool:
    if not cluster_available():
        return False
    f = fn("gemm_tcgen05_cluster", "rf_gemm_tc_cluster_supported", [c_int, c_int, c_int, c_int])
    return bool(f(M, N, K, mode))


_cluster_width = {}


def cluster_width(cluster: int = 2) -> int:
    """Clusters of the persistent kernel that run at once on this device."""
    key = (cluster, cluster_pair())
    if key not in _cluster_width:
        f = fn("gemm_tcgen05_cluster", "rf_gemm_tc_cluster_width", [c_int])
        n = f(cluster)
        need(n > 0, f"the clustered kernel cannot be launched with clusters of {cluster} (code {n})")
        _cluster_width[key] = n
    return _cluster_width[key]


def set_cluster_pair(on: bool) -> None:
    """Clusters of two as one MMA unit (the even CTA issues 256-row products over both CTAs' shared and tensor
    memory) instead of two CTAs that multicast their halves of a weight tile to each other."""
    fn("gemm_tcgen05_cluster", "rf_gemm_tc_cluster_set_pair", [c_int])(1 if on else 0)


def cluster_pair() -> bool:
    return bool(fn("gemm_tcgen05_cluster", "rf_gemm_tc_cluster_pair", [])())


_part_flags = {}


def part_flags(device) -> torch.Tensor:
    """Counters of the clustered kernel's K parts (one per output tile): zeroed once, left zeroed by every launch."""
    key = torch.device(device).index or 0
    if key not in _part_flags:
        _part_flags[key] = torch.zeros((1 << 16,), dtype=torch.int32, device=device)
    return _part_flags[key]


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *, mode: int = STORE,
            out: Optional[torch.Tensor] = None, cluster: Optional[int] = None,
            parts: int = 0) -> torch.Tensor:
    """Tokens as accumulator rows (any M).  STORE -> bf16 [M,N]; F32 -> f32 [M,N]; RESIDUAL: out (f32) += x w^T;
    SWIGLU -> bf16 [M, N/2] from row-interleaved gate/up weights.  ``parts`` (clustered kernel, RESIDUAL only):
    K parts whose sums are added one after the other, 0 = the kernel's own choice."""
    _common(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    need(supported(M, N, K, mode), f"tensor-core gemm: shape {M}x{N}x{K} is not supported")
    cols = N // 2 if mode == SWIGLU else N
    odt = torch.bfloat16 if mode in (STORE, SWIGLU) else torch.float32
    if out is None:
        need(mode != RESIDUAL, "gemm: RESIDUAL needs the tensor to add into")
        out = torch.empty((M, cols), dtype=odt, device=x.device)
    need(out.shape == (M, cols) and out.dtype == odt and out.stride(1) == 1, "gemm: output has the wrong shape or dtype")
    if cluster is None:
        cluster = 2 if cluster_supported(M, N, K, mode) else 0      # 2 measured at least as fast as 4
    if cluster and not cluster_supported(M, N, K, mode):
        cluster = 0                                   # e.g. an output row stride TMA cannot store to
    need(parts == 0 or (bool(cluster) and mode == RESIDUAL), "gemm: K parts need the clustered kernel and RESIDUAL")
    if cluster:
        f = fn("gemm_tcgen05_cluster", "rf_gemm_tc_cluster",
               [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                c_int, c_void_p, c_int, c_void_p, c_void_p])
        flags = part_flags(x.device)
        check(f(ptr(x), x.stride(0), ptr(w), ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                ptr(out), out.stride(0), M, N, K, mode, cluster, parts, ptr(flags), flags.numel(),
                ptr(status_word(x.device)), stream()),
              f"gemm_tc_cluster ({M}x{N}x{K}, cluster {cluster})")
        return out
    f = _f("rf_gemm_tc", c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
           c_void_p, c_void_p)
    check(f(ptr(x), x.stride(0), ptr(w), ptr(bias), int(bias is not None and bias.dtype == torch.float32), ptr(out),
            out.stride(0), M, N, K, mode, ptr(status_word(x.device)), stream()), f"gemm_tc ({M}x{N}x{K})")
    return out


def split_k_for(N: int, K: int, sm_count: Optional[int] = None, tokens: Optional[int] = None) -> int:
    """K splits of a skinny product, from N and K (never from the batch's content), so that about two CTAs per SM stream
    the weight and every split keeps at least 4 blocks of 64.  ``tokens``: a step of at most 16 tokens fits three CTAs on an
    SM, and a weight with long K ranges is then cut for three per SM (splits of at least 16 blocks; the down projection of
    the 7B shape 10 -> 15: a decode step at batch 8 2.624 -> 2.603 ms, at batch 1 2.560 -> 2.530 ms; with 32 or 64 tokens,
    two CTAs per SM, the same cut costs 0.16 ms).  The short K ranges of q|k|v and o gain nothing from more splits."""
    sm_count = sm_count or device_sm_count()
    tiles = (N + 127) // 128
    kb = (K + 63) // 64
    if tiles >= 2 * sm_count or kb < 8:
        return 1
    want = max(1, (2 * sm_count) // tiles)
    splits = max(1, min(want, kb // 4))
    if tokens is not None and tokens <= 16:
        splits = max(splits, min((3 * sm_count) // tiles, kb // 16))
    per = (kb + splits - 1) // splits
    return (kb + per - 1) // per                   # no empty split


_EX_ARGS = (c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
            c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p)


def _row_ss_args(row_ss, M):
    """(pointer, tiles, stride, eps) of a deferred norm's sums of squares, or zeros."""
    if row_ss is None:
        return ptr(None), 0, 0, 0.0
    ss, eps = row_ss
    need(ss.dtype == torch.float32 and ss.dim() == 2 and ss.stride(1) == 1 and ss.shape[1] >= M and ss.is_cuda,
         "skinny gemm: sums of squares must be a float32 [tiles, >= M] tensor on the device")
    return ptr(ss), ss.shape[0], ss.stride(0), float(eps)


def gemm_tc_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *, mode: int = STORE,
                   splits: int = 1, out: Optional[torch.Tensor] = None, row_ss=None) -> torch.Tensor:
    """Weights as accumulator rows, for few tokens (up to 128 in one tile).  With ``splits`` > 1 the mode must be PARTIAL and
    the result is the float32 stack [splits, M, N] of partial sums.

    ``row_ss`` = (ss [tiles, >= M] float32, eps): ``x`` holds rows that still have to be divided by their RMS
    (see ``gemm_tc_skinny_resnorm``); output row m is scaled by rsqrt(sum_t ss[t, m] / K + eps)."""
    _common(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    need(M <= SKINNY_MAX_TOKENS, f"skinny gemm takes at most {SKINNY_MAX_TOKENS} tokens, got {M}")
    need(supported(M, N, K, mode), f"tensor-core gemm: shape {M}x{N}x{K} is not supported")
    need(mode != RESNORM, "skinny gemm: the fused residual + norm epilogue has its own function")
    need(splits == 1 or mode == PARTIAL, "skinny gemm: several K splits need mode PARTIAL")
    cols = N // 2 if mode == SWIGLU else N
    odt = torch.bfloat16 if mode in (STORE, SWIGLU) else torch.float32
    shape = (splits, M, N) if mode == PARTIAL else (M, cols)
    if out is None:
        need(mode != RESIDUAL, "gemm: RESIDUAL needs the tensor to add into")
        out = torch.empty(shape, dtype=odt, device=x.device)
    need(tuple(out.shape) == shape and out.dtype == odt and out.is_contiguous(), "gemm: output has the wrong shape or dtype")
    if row_ss is None:
        f = _f("rf_gemm_tc_skinny", c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
               c_int, c_int, c_void_p, c_void_p)
        check(f(ptr(x), x.stride(0), ptr(w), ptr(bias), int(bias is not None and bias.dtype == torch.float32), ptr(out),
                cols, M, N, K, mode, splits, ptr(status_word(x.device)), stream()), f"gemm_tc_skinny ({M}x{N}x{K})")
        return out
    f = _f("rf_gemm_tc_skinny_ex", *_EX_ARGS)
    ss_ptr, ss_tiles, ss_stride, eps = _row_ss_args(row_ss, M)
    check(f(ptr(x), x.stride(0), ptr(w), ptr(bias), int(bias is not None and bias.dtype == torch.float32), ptr(out),
            cols, M, N, K, mode, splits, ss_ptr, ss_tiles, ss_stride, eps, ptr(None), ptr(None), 0, ptr(None), ptr(None), 0,
            ptr(status_word(x.device)), stream()), f"gemm_tc_skinny ({M}x{N}x{K}, rows scaled)")
    return out


def resnorm_splits(N: int, K: int) -> int:
    """K splits of the product that finishes the residual update itself: the splits of a tile are one thread-block
    cluster, so a power of two up to 8, as near the ordinary rule as that allows; from N and K alone."""
    want = split_k_for(N, K)
    kb = (K + 63) // 64
    s = 1
    while s * 2 <= min(want, 8) and (s * 2 - 1) * ((kb + s * 2 - 1) // (s * 2)) < kb:
        s *= 2
    return s


def gemm_tc_skinny_resnorm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], h: torch.Tensor,
                           norm_weight: torch.Tensor, splits: int = 1, row_ss=None):
    """h += x w^T (+ bias) for few tokens, and the next RMS norm prepared in the same launch.

    The product is split over K; the ``splits`` (1, 2, 4 or 8) CTAs of an output tile form a thread-block cluster, each
    owns a share of the tile's tokens, receives the others' partial sums of those tokens in its shared memory, adds
    them in rank order (so the result does not depend on timing) and the bias into the 32-bit stream ``h`` [M, N], and
    writes ``normed`` [M, N] = h * norm_weight in bfloat16 and ``ss`` [ceil(N/128), M], each weight tile's sum of h^2
    per token.  Whoever multiplies ``normed`` by a matrix next scales its output rows by
    rsqrt(sum_t ss[t, m] / N + eps) (``row_ss`` of ``gemm_tc_skinny``), which completes the norm.  Returns (normed, ss)."""
    _common(x, w, bias, None)
    need_cuda(h, norm_weight)
    M, K = x.shape
    N = w.shape[0]
    need(M <= SKINNY_MAX_TOKENS, f"skinny gemm takes at most {SKINNY_MAX_TOKENS} tokens, got {M}")
    need(supported(M, N, K, RESNORM), f"tensor-core gemm: shape {M}x{N}x{K} is not supported")
    need(h.dtype == torch.float32 and tuple(h.shape) == (M, N) and h.is_contiguous(), "resnorm: h must be float32 [M, N]")
    need(norm_weight.shape == (N,) and norm_weight.dtype in (torch.float32, torch.bfloat16), "resnorm: norm weight must be [N]")
    need(splits in (1, 2, 4, 8), "resnorm: 1, 2, 4 or 8 K splits (they form a thread-block cluster)")
    tiles = (N + 127) // 128
    normed = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    ss = torch.empty((tiles, M), dtype=torch.float32, device=x.device)
    f = _f("rf_gemm_tc_skinny_ex", *_EX_ARGS)
    ss_ptr, ss_tiles, ss_stride, eps = _row_ss_args(row_ss, M)
    check(f(ptr(x), x.stride(0), ptr(w), ptr(bias), int(bias is not None and bias.dtype == torch.float32), ptr(None),
            N, M, N, K, RESNORM, splits, ss_ptr, ss_tiles, ss_stride, eps, ptr(h), ptr(norm_weight),
            int(norm_weight.dtype == torch.float32), ptr(normed), ptr(ss), ss.stride(0),
            ptr(status_word(x.device)), stream()), f"gemm_tc_skinny_resnorm ({M}x{N}x{K})")
    return normed, ss
