from .spec import ParamSpec
from .safetensors_io import ModelFiles, SafetensorsFile, SafetensorsError, write_safetensors
from .loader import WeightError, load_folder, check_folder, target_dtype
from .random_init import random_tensors, random_tensor, write_model_folder
