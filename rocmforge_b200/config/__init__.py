from .errors import ConfigError, MissingKey, InvalidValue, UnknownArchitecture
from .registry import (register_architecture, architecture_for, known_architectures,
                       load_config, read_config_json, architecture_name)
from .qwen2 import Qwen2Config
