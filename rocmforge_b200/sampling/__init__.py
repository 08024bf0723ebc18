from .params import SamplingParams, draw_seed, as_int64, DEFAULT_SEED, REQUEST_STRIDE
from .device_sampler import DeviceSampler
