from ._ffi import KernelError
from .basic import (PAGE, embed, add_rmsnorm, rope_kv_write, swiglu, gemm_simt, split_k_for_simt, attention_generic, argmax, sample, set_sample_cached, advance_decode, gather_tokens,
                    attention_decode, attention_decode_supported, attention_decode_scratch, DECODE_CHUNK,
                    attention_prefill, attention_prefill_supported, PREFILL_TILE,
                    attention_decode_warps, decode_splits, decode_pages,
                    attention_prefill_tc, attention_prefill_tc_supported, PREFILL_TC_TILE)
from ._ffi import launch_count
from . import tensor_core
