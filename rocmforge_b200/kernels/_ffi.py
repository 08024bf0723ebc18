"""Glue between torch tensors and the ``extern "C"`` launchers of ``csrc``."""
from __future__ import annotations

import ctypes

import torch

from ..csrc import build

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


class KernelError(RuntimeError):
    pass


_CODES = {-1: "bad argument", -2: "size not supported by this kernel",
          -3: "device error flag set by the kernel (a bounded wait ran out)"}


_launches = 0


def launch_count() -> int:
    """How many launcher calls of this package's CUDA modules succeeded so far in this process."""
    return _launches


def check(code: int, what: str) -> None:
    global _launches
    if code == 0:
        _launches += 1
        return
    if code < 0:
        raise KernelError(f"{what}: {_CODES.get(code, f'error {code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return 0
    if dt == torch.bfloat16:
        return 1
    raise KernelError(f"compute dtype {dt} is not supported (float32 or bfloat16)")


def ptr(t) -> c_void_p:
    return c_void_p(0) if t is None else c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> c_void_p:
    """torch's current stream of the current device as a raw handle.  Asked at every launch (the current
    stream changes under ``torch.cuda.stream`` and during graph capture), so through the cheapest call there is:
    ``torch.cuda.current_stream()`` builds a Stream object and costs about 15 us, a third of a launch's host time."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("rocmforge_b200 kernels run on a CUDA device only; got a tensor on "
                              f"{t.device} (there is no CPU fallback)")


def need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def fn(module: str, name: str, argtypes):
    lib = build.load(module)
    f = getattr(lib, name)
    f.argtypes = argtypes
    f.restype = c_int
    return f


_sm_count = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (148 on a B200): launch shapes are sized by it, not by a constant.
    Without a CUDA device (host-side tests of the launch rules) the B200's number stands in."""
    if not torch.cuda.is_available():
        return 148
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]
