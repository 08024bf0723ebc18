"""One registry from an architecture's name to its configuration class and model builder.

maeddesg/ROCmForge looks a GGUF architecture string up in a traits table and falls
back to LLaMA behaviour for unknown names (src/config.rs:515-517).  Here the key is
``architectures[0]`` of config.json and an unknown name is an error.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict

from .errors import ConfigError, MissingKey, UnknownArchitecture


@dataclass
class Architecture:
    name: str
    config_cls: type              # has from_dict(dict) -> config
    build: Callable               # build(config) -> engine.model.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, build: Callable) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_cls, build)


def known_architectures():
    return sorted(_ARCHITECTURES)


def architecture_for(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise UnknownArchitecture(name, _ARCHITECTURES.keys())
    return _ARCHITECTURES[name]


def architecture_name(raw: dict) -> str:
    archs = raw.get("architectures")
    if not archs:
        raise MissingKey("architectures")
    if not isinstance(archs, (list, tuple)) or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a list of names")
    return archs[0]


def read_config_json(folder_or_file: str) -> dict:
    path = folder_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.exists(path):
        raise ConfigError(f"no config.json at {path}")
    with open(path) as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw


def load_config(folder_or_file: str):
    """config.json -> (Architecture, typed configuration)."""
    raw = read_config_json(folder_or_file)
    arch = architecture_for(architecture_name(raw))
    return arch, arch.config_cls.from_dict(raw)
