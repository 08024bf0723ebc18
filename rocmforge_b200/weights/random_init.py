"""Random weights from a configuration and a seed.

maeddesg/ROCmForge has no such mode (its whole-model tests need downloaded files,
tests/gpu_decode_real.rs:20-21).  Matrices and biases are normal with the spec's
standard deviation, norm weights are one.  An element's value is a function of
(seed, tensor name, element index) alone: it does not depend on which other tensors
exist, on the device that makes it, or on how the work is cut.  The host (torch integer
and float64 operations) and the device (csrc/random_fill.cu) carry out the same
arithmetic operation for operation, so ``Model.random(config, seed)`` on the GPU and
``write_model_folder(..., seed)`` on the host are the same model bit for bit.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Iterator, Tuple

import torch

from .safetensors_io import write_safetensors
from .spec import ParamSpec


MASK64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15
_C1, _C2 = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
CELLS = 1 << 16


def _signed(u: int) -> int:
    """The 64 bits of ``u`` as a signed integer (torch has no unsigned 64-bit arithmetic; sums and products wrap alike)."""
    u &= MASK64
    return u - (1 << 64) if u >= (1 << 63) else u


def _mix64_int(z: int) -> int:
    z &= MASK64
    z = ((z ^ (z >> 30)) * _C1) & MASK64
    z = ((z ^ (z >> 27)) * _C2) & MASK64
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """64-bit key of a tensor's random stream, from the seed and the tensor's name."""
    data = name.encode("utf-8")
    h = _mix64_int(int(seed) & MASK64)
    h = _mix64_int(h ^ zlib.crc32(data) ^ (zlib.adler32(data) << 32))
    return h


_table = {}


def normal_table(device="cpu") -> torch.Tensor:
    """Standard normal quantiles at the probabilities i / 65536, i = 0 .. 65536 (the ends moved in to 2^-17 and
    1 - 2^-17), float64: the knots of a piecewise linear inverse distribution function.  Computed once on the host
    and copied to a device, so that both sides read the same numbers."""
    if "cpu" not in _table:
        p = torch.arange(CELLS + 1, dtype=torch.float64) / CELLS
        p = p.clamp(2.0 ** -17, 1.0 - 2.0 ** -17)
        _table["cpu"] = torch.special.ndtri(p)
    key = str(torch.device(device))
    if key not in _table:
        _table[key] = _table["cpu"].to(device)
    return _table[key]


def _lsr(z: torch.Tensor, k: int) -> torch.Tensor:
    return (z >> k) & ((1 << (64 - k)) - 1)          # logical shift of the 64 bits held in a signed tensor


def fill_normal_host(n: int, key: int, std: float, dtype: torch.dtype, chunk: int = 1 << 24) -> torch.Tensor:
    """n values of the stream ``key`` on the host: the device kernel's arithmetic with torch operations."""
    table = normal_table("cpu")
    out = torch.empty((n,), dtype=dtype)
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        z = torch.arange(lo + 1, hi + 1, dtype=torch.int64) * _signed(GOLDEN) + _signed(key)
        z = (z ^ _lsr(z, 30)) * _signed(_C1)
        z = (z ^ _lsr(z, 27)) * _signed(_C2)
        z = z ^ _lsr(z, 31)
        u = _lsr(z, 32)
        cell = u >> 16
        frac = (u & 0xFFFF).to(torch.float64) * (1.0 / 65536.0)
        a, b = table[cell], table[cell + 1]
        d = b - a
        d = frac * d                                  # product and sum rounded one after the other, as on the device
        v = (a + d) * float(std)
        out[lo:hi] = v.to(torch.float32).to(dtype)
    return out


def fill_normal_device(n: int, key: int, std: float, dtype: torch.dtype, device) -> torch.Tensor:
    import ctypes
    from ..kernels._ffi import check, dtype_code, fn, ptr, stream
    out = torch.empty((n,), dtype=dtype, device=device)
    table = normal_table(device)
    f = fn("random_fill", "rf_fill_normal", [ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_ulonglong,
                                             ctypes.c_double, ctypes.c_void_p, ctypes.c_void_p])
    with torch.cuda.device(out.device):
        check(f(dtype_code(dtype), ptr(out), n, key & MASK64, float(std), ptr(table), stream()), "fill_normal")
    return out


def random_tensor(name: str, spec: ParamSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    if spec.init == "ones":
        return torch.ones(spec.shape, dtype=dtype, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    n = 1
    for d in spec.shape:
        n *= int(d)
    key = tensor_key(seed, name)
    if spec.kind == "int_table":                       # 15-bit integers from the same stream of bits
        z = torch.arange(1, n + 1, dtype=torch.int64) * _signed(GOLDEN) + _signed(key)
        z = (z ^ _lsr(z, 30)) * _signed(_C1)
        z = (z ^ _lsr(z, 27)) * _signed(_C2)
        z = z ^ _lsr(z, 31)
        return (_lsr(z, 49)).to(torch.int32).reshape(spec.shape).to(device)
    if dtype not in (torch.float32, torch.bfloat16):
        return fill_normal_host(n, key, spec.std, torch.float32).to(dtype).reshape(spec.shape).to(device)
    if torch.device(device).type == "cuda":
        return fill_normal_device(n, key, spec.std, dtype, device).reshape(spec.shape)
    return fill_normal_host(n, key, spec.std, dtype).reshape(spec.shape)


def random_tensors(specs: Dict[str, ParamSpec], seed: int, dtype: torch.dtype,
                   device="cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    """(name, tensor) for every spec that is not left to its tied partner."""
    for name, spec in specs.items():
        if spec.tied_to is not None:
            continue
        yield name, random_tensor(name, spec, seed, dtype, device)


def write_model_folder(folder: str, config_dict: dict, specs: Dict[str, ParamSpec], seed: int,
                       dtype: torch.dtype = torch.bfloat16, device="cpu") -> None:
    """config.json and model.safetensors of a randomly initialised model.  ``device``: where the values are made
    (the same values either way; a GPU makes a large model in seconds)."""
    os.makedirs(folder, exist_ok=True)
    cfg = dict(config_dict)
    cfg["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                          torch.float16: "float16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      ((name, t.cpu()) for name, t in random_tensors(specs, seed, dtype, device)),
                      metadata={"format": "pt", "seed": seed})
