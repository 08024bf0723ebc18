from ._ffi import KernelError
from .basic import (PAGE, embed, add_rmsnorm, rope_kv_write, swiglu, gemm_simt, attention_generic, argmax, sample, advance_decode)
from ._ffi import launch_count
from . import tensor_core
