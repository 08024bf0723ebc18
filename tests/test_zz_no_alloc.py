"""The allocation-free decode attention, called through its exported C symbol (needs a GPU).

Some users of this library run where device memory may not be allocated: a plug-in inside a
serving process that owns every byte of the GPU, or a thread that must never wait on the
allocator.  For them ``rf_attention_decode_noalloc`` keeps the kernel's scratch space in a fixed
8 MiB array inside the library itself.  This test loads the shared library with ctypes, as such a
caller would, runs the entry point twice in a row on the same inputs (the second call finds the
array as the first one left it) and compares both results with the ordinary entry point, which
takes its scratch from the caller, and with an attention written out here in float64.  It also
checks that a request larger than the fixed array is refused instead of being run, and that a
sequence longer than the chunks the caller announced is reported and left alone.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(nh, nkv, hd, lens, seed=0):
    """Random queries and a paged bfloat16 cache holding sequences of the given lengths (pages shuffled, the
    unused rest of every page NaN).  Returns the device tensors and the keys and values per sequence."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    pages_per = [(n + 63) // 64 for n in lens]
    n_pages = sum(pages_per) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(B, max(pages_per) + 1, dtype=torch.int32)
    k_pages = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=torch.bfloat16)
    v_pages = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=torch.bfloat16)
    ks, vs = [], []
    for s, n in enumerate(lens):
        k = torch.randn(n, nkv, hd, generator=g).bfloat16()
        v = torch.randn(n, nkv, hd, generator=g).bfloat16()
        ks.append(k); vs.append(v)
        for p in range(pages_per[s]):
            page = order.pop()
            table[s, p] = page
            m = min(64, n - 64 * p)
            k_pages[page, :, :m] = k[64 * p:64 * p + m].transpose(0, 1)
            v_pages[page, :, :m] = v[64 * p:64 * p + m].transpose(0, 1)
    q = torch.randn(B, nh * hd, generator=g).bfloat16()
    ints = dict(tok_seq=torch.arange(B, dtype=torch.int32), tok_pos=torch.tensor([n - 1 for n in lens], dtype=torch.int32),
                seq_slot=torch.arange(B, dtype=torch.int32))
    return (q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), table.to(DEV), {k: v.to(DEV) for k, v in ints.items()}), (q, ks, vs)


def _plain_attention(q, ks, vs, lens, nh, nkv, hd, scale, window):
    """softmax(q k^T * scale) v in float64 for the newest position of every sequence (last ``window`` keys)."""
    out = torch.zeros(len(lens), nh, hd, dtype=torch.float64)
    for b, n in enumerate(lens):
        lo = 0 if not window else max(0, n - window)
        for h in range(nh):
            kh = h // (nh // nkv)
            s = (ks[b][lo:n, kh].double() @ q[b].view(nh, hd)[h].double()) * scale
            out[b, h] = torch.softmax(s, dim=0) @ vs[b][lo:n, kh].double()
    return out.view(len(lens), nh * hd)


def _entry_point():
    from rocmforge_b200.csrc import build
    build.ensure_built(["attention_decode_noalloc"])
    lib = ctypes.CDLL(build.lib_path("attention_decode_noalloc"))
    f = lib.rf_attention_decode_noalloc
    vp, i, fl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    f.argtypes = [vp, i, vp, i, vp, vp, vp, vp, vp, vp, i, i, i, i, fl, i, i, i, vp, vp]
    f.restype = i
    return f


@pytest.mark.parametrize("window", [0, 300])
def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(window):
    """Sequences that end on a page border (64), on a chunk border (128) and just behind it (129) among others,
    with all keys and with a window of 300: both calls equal the ordinary entry point and a float64 attention
    written out here, the two calls equal each other bit for bit (the merge order is fixed), and the free device
    memory that the driver reports does not move across the second call."""
    from rocmforge_b200 import kernels
    nh, nkv, hd = 28, 4, 128
    lens = [700, 1, 129, 512, 64, 128]
    B, max_chunks = len(lens), 8
    (q, k_pages, v_pages, table, ints), (q_h, ks, vs) = _inputs(nh, nkv, hd, lens)
    scale = 1.0 / math.sqrt(hd)
    plain = _plain_attention(q_h, ks, vs, lens, nh, nkv, hd, scale, window)
    n_o, n_ml, n_c = kernels.attention_decode_scratch(B, nh, nkv, hd, max_chunks)
    want = kernels.attention_decode(q, nh, nkv, hd, k_pages, v_pages, ints["tok_seq"], ints["tok_pos"], ints["seq_slot"],
                                    table, scale, window or None, max_chunks, torch.zeros(n_o, device=DEV),
                                    torch.zeros(n_ml, device=DEV), torch.zeros(n_c, dtype=torch.int32, device=DEV))
    f = _entry_point()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    outs = [torch.full((B, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    for call, out in enumerate(outs):
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()           # what the driver has left, whoever allocates
        rc = f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
               ints["tok_seq"].data_ptr(), ints["tok_pos"].data_ptr(), ints["seq_slot"].data_ptr(), table.data_ptr(),
               table.shape[1], nh, nkv, hd, scale, window, B, max_chunks, status.data_ptr(), stream)
        assert rc == 0, f"call {call}: the entry point returned {rc}"
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        if call == 1:        # the first call on a device may make the runtime load the kernel's image
            assert free_after == free_before, f"device memory moved by {free_before - free_after} bytes across the call"
        assert int(status.item()) == 0
        assert torch.isfinite(out.float()).all(), f"call {call}: part of the output was not written"
        torch.testing.assert_close(out.float(), want.float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(out.double().cpu(), plain, atol=2e-2, rtol=2e-2)
    assert torch.equal(outs[0], outs[1]), "the second call found the array changed and gave another result"


def test_no_alloc_entry_point_reports_a_sequence_beyond_its_chunks():
    """``max_chunks`` must cover the longest sequence; one that is longer is reported in the status word and the
    output stays as it was (nothing is read or written out of bounds)."""
    nh, nkv, hd = 8, 2, 64
    (q, k_pages, v_pages, table, ints), _ = _inputs(nh, nkv, hd, [300, 40])
    f = _entry_point()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((2, nh * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
           ints["tok_seq"].data_ptr(), ints["tok_pos"].data_ptr(), ints["seq_slot"].data_ptr(), table.data_ptr(),
           table.shape[1], nh, nkv, hd, 0.125, 0, 2, 2, status.data_ptr(), stream)       # 2 chunks = 256 keys < 300
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 3
    assert (out[0] == 7.0).all(), "the sequence without a CTA for its last chunk must be left alone"
    assert torch.isfinite(out[1].float()).all() and not (out[1] == 7.0).all()


def test_no_alloc_entry_point_refuses_more_than_its_array_holds():
    nh, nkv, hd = 28, 4, 128
    (q, k_pages, v_pages, table, ints), _ = _inputs(nh, nkv, hd, [5, 9])
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
