"""Weights by tensor name, from a model folder to the device.

Counterpart of maeddesg/ROCmForge's ``GpuModelWeights::load`` (src/gpu/weights.rs:830-928):
every tensor the model's parts ask for is looked up by its name; unlike the reference,
which stops at the first tensor it cannot find (src/gpu/weights.rs:567-574), all faults
of a folder are collected into ONE error that lists missing tensors, unexpected ones
and wrong shapes.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from .safetensors_io import ModelFiles
from .spec import ParamSpec


class WeightError(ValueError):
    """The folder's tensors do not fit the model: see .missing, .unexpected, .wrong_shape, .wrong_dtype."""

    def __init__(self, folder, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing: List[str] = sorted(missing)
        self.unexpected: List[str] = sorted(unexpected)
        self.wrong_shape: List[Tuple[str, tuple, tuple]] = sorted(wrong_shape)
        self.wrong_dtype: List[Tuple[str, str]] = sorted(wrong_dtype)
        lines = [f"weights in {folder} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, the configuration needs {list(want)}")
        for name, why in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name}: {why}")
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


def target_dtype(spec: ParamSpec, stored: torch.dtype, compute_dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in on the device."""
    if spec.kind == "int_table":
        return torch.int32
    if compute_dtype == torch.float32:
        return torch.float32
    if spec.kind == "vector":
        # a tensor stored in 32-bit stays so; one stored in 16-bit is kept in bfloat16
        return torch.float32 if stored in (torch.float32, torch.float64) else torch.bfloat16
    return compute_dtype


def check_folder(files: ModelFiles, specs: Dict[str, ParamSpec]) -> None:
    """Raise one WeightError if names, shapes or dtype classes do not fit ``specs``."""
    missing, unexpected, wrong_shape, wrong_dtype = [], [], [], []
    have = set(files.names())
    for name, spec in specs.items():
        if name not in have:
            if spec.tied_to is not None and spec.tied_to in have:
                continue
            missing.append(name)
            continue
        e = files.entries[name]
        if tuple(e.shape) != tuple(spec.shape):
            wrong_shape.append((name, tuple(e.shape), tuple(spec.shape)))
        if spec.kind == "int_table" and e.dtype not in _INTS:
            wrong_dtype.append((name, f"stored as {e.dtype}, an integer table is needed"))
        if spec.kind != "int_table" and e.dtype not in _FLOATS:
            wrong_dtype.append((name, f"stored as {e.dtype}, a floating-point tensor is needed"))
    for name in have:
        if name not in specs:
            unexpected.append(name)
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(files.folder, missing, unexpected, wrong_shape, wrong_dtype)


def load_folder(folder: str, specs: Dict[str, ParamSpec], compute_dtype: torch.dtype,
                device) -> Dict[str, torch.Tensor]:
    """{name: device tensor} for every name in ``specs``; tied tensors share storage."""
    files = ModelFiles(folder)
    check_folder(files, specs)
    out: Dict[str, torch.Tensor] = {}
    have = set(files.names())
    for name, spec in specs.items():
        if name not in have:
            continue
        src = files.tensor(name)
        out[name] = src.to(device=device, dtype=target_dtype(spec, src.dtype, compute_dtype)).contiguous()
    for name, spec in specs.items():
        if name not in out:
            # src/gpu/weights.rs:868-886 makes a second copy for a tied head; an alias is enough
            out[name] = out[spec.tied_to]
    return out
