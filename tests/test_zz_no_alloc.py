"""The allocation-free decode attention, called through its exported C symbol (needs a GPU).

Some users of this library run where device memory may not be allocated: a plug-in inside a
serving process that owns every byte of the GPU, or a thread that must never wait on the
allocator.  For them ``rf_attention_decode_noalloc`` keeps the kernel's scratch space in a fixed
8 MiB array inside the library itself.  This test loads the shared library with ctypes, as such a
caller would, runs the entry point twice in a row on the same inputs (the second call finds the
array as the first one left it) and compares both results with the ordinary entry point, which
takes its scratch from the caller.  It also checks that a request larger than the fixed array is
refused instead of being run.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(nh, nkv, hd, lens, seed=0):
    """Random queries and a paged bfloat16 cache holding sequences of the given lengths."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    pages_per = [(n + 63) // 64 for n in lens]
    n_pages = sum(pages_per) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(B, max(pages_per) + 1, dtype=torch.int32)
    k_pages = torch.zeros(n_pages, nkv, 64, hd, dtype=torch.bfloat16)
    v_pages = torch.zeros(n_pages, nkv, 64, hd, dtype=torch.bfloat16)
    for s, n in enumerate(lens):
        for p in range(pages_per[s]):
            page = order.pop()
            table[s, p] = page
            m = min(64, n - 64 * p)
            k_pages[page, :, :m] = torch.randn(nkv, m, hd, generator=g).bfloat16()
            v_pages[page, :, :m] = torch.randn(nkv, m, hd, generator=g).bfloat16()
    q = torch.randn(B, nh * hd, generator=g).bfloat16()
    ints = dict(tok_seq=torch.arange(B, dtype=torch.int32), tok_pos=torch.tensor([n - 1 for n in lens], dtype=torch.int32),
                seq_slot=torch.arange(B, dtype=torch.int32))
    return (q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), table.to(DEV), {k: v.to(DEV) for k, v in ints.items()})


def _entry_point():
    from rocmforge_b200.csrc import build
    build.ensure_built(["attention_decode_noalloc"])
    lib = ctypes.CDLL(build.lib_path("attention_decode_noalloc"))
    f = lib.rf_attention_decode_noalloc
    vp, i, fl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    f.argtypes = [vp, i, vp, i, vp, vp, vp, vp, vp, vp, i, i, i, i, fl, i, i, i, vp, vp]
    f.restype = i
    return f


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from rocmforge_b200 import kernels
    nh, nkv, hd = 28, 4, 128
    lens = [700, 1, 129, 512, 64]
    B, max_chunks = len(lens), 8
    q, k_pages, v_pages, table, ints = _inputs(nh, nkv, hd, lens)
    scale = 1.0 / math.sqrt(hd)
    n_o, n_ml, n_c = kernels.attention_decode_scratch(B, nh, nkv, hd, max_chunks)
    want = kernels.attention_decode(q, nh, nkv, hd, k_pages, v_pages, ints["tok_seq"], ints["tok_pos"], ints["seq_slot"],
                                    table, scale, None, max_chunks, torch.zeros(n_o, device=DEV),
                                    torch.zeros(n_ml, device=DEV), torch.zeros(n_c, dtype=torch.int32, device=DEV))
    f = _entry_point()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    for call in range(2):
        out = torch.full((B, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        held = torch.cuda.memory_allocated()
        rc = f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
               ints["tok_seq"].data_ptr(), ints["tok_pos"].data_ptr(), ints["seq_slot"].data_ptr(), table.data_ptr(),
               table.shape[1], nh, nkv, hd, scale, 0, B, max_chunks, status.data_ptr(), stream)
        assert rc == 0, f"call {call}: the entry point returned {rc}"
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == held, "the call went through torch's allocator"
        assert int(status.item()) == 0
        assert torch.isfinite(out.float()).all(), f"call {call}: part of the output was not written"
        torch.testing.assert_close(out.float(), want.float(), atol=2e-2, rtol=2e-2)
    assert before <= torch.cuda.memory_allocated()


def test_no_alloc_entry_point_refuses_more_than_its_array_holds():
    nh, nkv, hd = 28, 4, 128
    q, k_pages, v_pages, table, ints = _inputs(nh, nkv, hd, [5, 9])
    f = _entry_point()
    out = torch.zeros(2, nh * hd, dtype=torch.bfloat16, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
            ints["tok_seq"].data_ptr(), ints["tok_pos"].data_ptr(), ints["seq_slot"].data_ptr(), table.data_ptr(),
            table.shape[1], nh, nkv, hd, 0.1, 0]
    # 64 sequences x 28 heads x 128 chunks x 130 floats = 119 MB of scratch: far beyond 8 MiB
    assert f(*args, 64, 128, None, stream) == -2
    assert f(*args, 2, 4, None, stream) == 0          # the same inputs at a size that fits still run
    torch.cuda.synchronize()
