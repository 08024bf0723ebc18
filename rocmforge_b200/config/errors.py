"""Typed errors of the configuration layer.

maeddesg/ROCmForge distinguishes a missing key from an invalid value
(src/config.rs:763-787); so does this module, and every message names the key.
"""


class ConfigError(ValueError):
    """Base class: something is wrong with config.json."""


class MissingKey(ConfigError):
    def __init__(self, key: str):
        super().__init__(f"config.json: required key '{key}' is missing")
        self.key = key


class InvalidValue(ConfigError):
    def __init__(self, key: str, value, why: str):
        super().__init__(f"config.json: key '{key}' = {value!r} is invalid: {why}")
        self.key = key


class UnknownArchitecture(ConfigError):
    def __init__(self, name, known):
        super().__init__(
            f"config.json: architecture {name!r} is not registered (known: {sorted(known)})")
        self.name = name
