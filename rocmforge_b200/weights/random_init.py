"""Random weights from a configuration and a seed.

maeddesg/ROCmForge has no such mode (its whole-model tests need downloaded files,
tests/gpu_decode_real.rs:20-21).  Matrices and biases are normal with the spec's
standard deviation, norm weights are one.  Each tensor has its own generator seeded
by (seed, tensor name), so a tensor's values do not depend on which other tensors exist.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Iterator, Tuple

import torch

from .safetensors_io import write_safetensors
from .spec import ParamSpec


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 1000003 + zlib.crc32(name.encode("utf-8"))) % (1 << 62)


def random_tensor(name: str, spec: ParamSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    if spec.kind == "int_table":
        g = torch.Generator(device=device).manual_seed(_tensor_seed(seed, name))
        return torch.randint(0, 1 << 15, spec.shape, generator=g, device=device, dtype=torch.int32)
    if spec.init == "ones":
        return torch.ones(spec.shape, dtype=dtype, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    g = torch.Generator(device=device).manual_seed(_tensor_seed(seed, name))
    t = torch.empty(spec.shape, dtype=torch.float32 if torch.device(device).type == "cpu" else dtype,
                    device=device)
    t.normal_(0.0, spec.std, generator=g)
    return t.to(dtype)


def random_tensors(specs: Dict[str, ParamSpec], seed: int, dtype: torch.dtype,
                   device="cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    """(name, tensor) for every spec that is not left to its tied partner."""
    for name, spec in specs.items():
        if spec.tied_to is not None:
            continue
        yield name, random_tensor(name, spec, seed, dtype, device)


def write_model_folder(folder: str, config_dict: dict, specs: Dict[str, ParamSpec], seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> None:
    """config.json and model.safetensors of a randomly initialised model."""
    os.makedirs(folder, exist_ok=True)
    cfg = dict(config_dict)
    cfg["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                          torch.float16: "float16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(specs, seed, dtype), metadata={"format": "pt", "seed": seed})
