"""rocmforge_b200: a small, whole generation library for one GPU (NVIDIA B200, sm_100a).

From a model folder (config.json + safetensors) or a configuration and a seed, through a
paged per-sequence cache and one step function, to sampled tokens; every hot operation is
a hand-written CUDA kernel, with a true 32-bit path beside the bfloat16 one.
"""
from . import models as _models          # fills the architecture registry
from .config import load_config, Qwen2Config, ConfigError
from .engine import Model, ModelSpec, ScheduleEntry, StepRequest, Options
from .cache import SequenceCache, CacheError
from .weights import WeightError, write_model_folder
from .sampling import SamplingParams
from .api import LLM
from .engine.generate import generate, GenerationResult

__all__ = ["load_config", "Qwen2Config", "ConfigError", "Model", "ModelSpec", "ScheduleEntry",
           "StepRequest", "Options", "LLM", "SamplingParams", "generate", "GenerationResult", "SequenceCache", "CacheError", "WeightError", "write_model_folder"]
