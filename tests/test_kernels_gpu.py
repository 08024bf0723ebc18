"""Each kernel alone against a plain PyTorch float64 reference of the same operation, at sizes
other than the tiny models' (needs a GPU)."""
import math

import numpy as np
import pytest
import torch

from plain import qwen2_plain as P
from plain import sampling_plain as S

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTS = [torch.float32, torch.bfloat16]


def tol(dt):
    return dict(atol=1e-5, rtol=1e-5) if dt == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def rnd(*shape, dt=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dt).to(DEV)


@pytest.mark.parametrize("dt", DTS)
def test_embed(dt):
    from rocmforge_b200 import kernels
    table = rnd(1000, 136, dt=dt)
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32, device=DEV)
    out = kernels.embed(table, ids)
    assert out.dtype == torch.float32 and torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H", [24, 1000, 3584, 5120])
def test_add_rmsnorm(dt, H):
    from rocmforge_b200 import kernels
    T = 7
    h = rnd(T, H, seed=1)
    for wdt in (torch.float32, torch.bfloat16):
        w = rnd(H, dt=wdt, seed=2) + 1.0
        # no pending
        h0 = h.clone()
        y = kernels.add_rmsnorm(h0, w, 1e-5, dt)
        ref = P.rms_norm(h.double(), w.double(), 1e-5)
        assert torch.equal(h0, h) and y.dtype == dt
        torch.testing.assert_close(y.double(), ref, **tol(dt))
        # split partial sums, added in 32-bit and written back
        parts = rnd(3, T, H, seed=3)
        h1 = h.clone()
        y = kernels.add_rmsnorm(h1, w, 1e-5, dt, pending=parts)
        total = h.double() + parts.double().sum(0)
        torch.testing.assert_close(h1.double(), total, atol=1e-5, rtol=1e-6)
        torch.testing.assert_close(y.double(), P.rms_norm(total, w.double(), 1e-5), **tol(dt))
        # pending in the compute dtype
        pend = rnd(T, H, dt=dt, seed=4)
        h2 = h.clone()
        y = kernels.add_rmsnorm(h2, w, 1e-5, dt, pending=pend)
        total = h.double() + pend.double()
        torch.testing.assert_close(h2.double(), total, atol=1e-5, rtol=1e-6)
        torch.testing.assert_close(y.double(), P.rms_norm(total, w.double(), 1e-5), **tol(dt))
        # rows: only those rows, h untouched
        rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
        h3 = h.clone()
        y = kernels.add_rmsnorm(h3, w, 1e-5, dt, pending=pend, rows=rows)
        assert torch.equal(h3, h) and tuple(y.shape) == (3, H)
        torch.testing.assert_close(y.double(), P.rms_norm(total[rows.long()], w.double(), 1e-5), **tol(dt))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H", [24, 1000, 3584, 5120, 9000])
def test_add_rmsnorm_of_a_prompt_step(dt, H):
    """Many rows without a pending update take a kernel of their own (rows read twice, the second time from L1); with a
    pending update or a row gather the other one.  All against the plain norm; the two kernels differ by the order of a
    row's sum of squares at most."""
    from rocmforge_b200 import kernels
    T = 700
    h = rnd(T, H, seed=11)
    for wdt in (torch.float32, torch.bfloat16):
        w = rnd(H, dt=wdt, seed=12) + 1.0
        h0 = h.clone()
        y = kernels.add_rmsnorm(h0, w, 1e-6, dt)
        assert torch.equal(h0, h) and tuple(y.shape) == (T, H) and y.dtype == dt
        torch.testing.assert_close(y.double(), P.rms_norm(h.double(), w.double(), 1e-6), **tol(dt))
        # the same rows with a zero update: the kernel that keeps a row in registers
        y2 = kernels.add_rmsnorm(h.clone(), w, 1e-6, dt, pending=torch.zeros(1, T, H, device=DEV))
        torch.testing.assert_close(y2.float(), y.float(), atol=1e-6 if dt == torch.float32 else 2e-2, rtol=1e-6 if dt == torch.float32 else 1e-2)
        rows = torch.arange(0, T, 7, dtype=torch.int32, device=DEV)
        y3 = kernels.add_rmsnorm(h.clone(), w, 1e-6, dt, rows=rows)
        torch.testing.assert_close(y3.double(), P.rms_norm(h[rows.long()].double(), w.double(), 1e-6), **tol(dt))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H", [896, 3584, 4100, 5120, 8192, 16384])
def test_add_rmsnorm_rows_shared_by_a_cluster_give_the_bits_of_one_block(dt, H):
    """With few rows a row's threads are spread over a thread-block cluster (up to 8 CTAs); with many rows one
    block works on a row.  Both must give the same bits, with and without partial sums, whatever the number of rows
    (a token's norm must not depend on the size of its batch)."""
    from rocmforge_b200 import kernels
    w = rnd(H, dt=torch.bfloat16, seed=2) + 1.0
    for n_pending in (0, 1, 3, 10, 17):     # from five on, small blocks ask for sixteen (eight) partial sums at once
        h = rnd(5, H, seed=5)
        parts = rnd(n_pending, 5, H, seed=6) if n_pending else None
        many_h, many_parts = h.repeat(80, 1), (parts.repeat(1, 80, 1) if n_pending else None)     # 400 rows: no clusters
        y_many = kernels.add_rmsnorm(many_h, w, 1e-6, dt, pending=many_parts)
        for n in (1, 2, 5):
            hn = h[:n].clone()
            yn = kernels.add_rmsnorm(hn, w, 1e-6, dt, pending=parts[:, :n].contiguous() if n_pending else None)
            assert torch.equal(yn, y_many[:n]), (H, n_pending, n)
            assert torch.equal(hn, many_h[:n])
        rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
        y_rows = kernels.add_rmsnorm(h.clone(), w, 1e-6, dt, pending=parts, rows=rows)
        assert torch.equal(y_rows, y_many[rows.long()])
        total = h.double() + (parts.double().sum(0) if n_pending else 0)
        torch.testing.assert_close(y_many[:5].double(), P.rms_norm(total, w.double(), 1e-6), **tol(dt))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (5, 130, 33), (65, 64, 64), (130, 200, 257), (3, 1000, 3584), (17, 896, 4864),
                                   (40, 300, 1000), (300, 1152, 896)])
def test_gemm_simt(dt, M, N, K):
    from rocmforge_b200 import kernels
    x, w = rnd(M, K, dt=dt, seed=1), rnd(N, K, dt=dt, seed=2, scale=0.1)
    bias = rnd(N, seed=3)
    ref = x.double() @ w.double().t()
    y = kernels.gemm_simt(x, w)
    assert y.dtype == dt
    # 32-bit sums of K products: the bound grows with K (maeddesg/ROCmForge allows 1e-4, tests/gpu_test_utils.rs:12)
    torch.testing.assert_close(y.double(), ref, **(dict(atol=1e-4, rtol=1e-5) if dt == torch.float32 else tol(dt)))
    y = kernels.gemm_simt(x, w, bias, out_f32=True)
    assert y.dtype == torch.float32
    torch.testing.assert_close(y.double(), ref + bias.double(), atol=1e-4, rtol=1e-5)
    acc = rnd(M, N, seed=4)
    acc0 = acc.clone()
    kernels.gemm_simt(x, w, out=acc, accumulate=True)
    torch.testing.assert_close(acc.double(), acc0.double() + ref, atol=1e-4, rtol=1e-5)
    # a row's result does not depend on the other rows of the batch, whatever tile height their number selects
    if M > 1:
        alone = kernels.gemm_simt(x[M - 1:M].contiguous(), w, out_f32=True)
        assert torch.equal(alone, kernels.gemm_simt(x, w, out_f32=True)[M - 1:M])
    # K ranges as partial sums: each split alone is the product over its range; their number follows N and K only
    kb = (K + 15) // 16
    for splits in {kernels.split_k_for_simt(N, K), (kb + (kb + 2) // 3 - 1) // ((kb + 2) // 3)}:       # the rule's, and about 3
        parts = kernels.gemm_simt(x, w, splits=splits)
        assert tuple(parts.shape) == (splits, M, N) and parts.dtype == torch.float32
        torch.testing.assert_close(parts.double().sum(0), ref, atol=1e-4, rtol=1e-5)
        per = ((K + 15) // 16 + splits - 1) // splits * 16
        for s in range(splits):
            lo, hi = s * per, min(K, (s + 1) * per)
            torch.testing.assert_close(parts[s].double(), x[:, lo:hi].double() @ w[:, lo:hi].double().t(), atol=1e-4, rtol=1e-5)
        if M > 1:
            assert torch.equal(kernels.gemm_simt(x[M - 1:M].contiguous(), w, splits=splits)[:, 0], parts[:, M - 1])


@pytest.mark.parametrize("dt", DTS)
def test_swiglu(dt):
    from rocmforge_b200 import kernels
    gu = rnd(9, 2 * 301, dt=dt, scale=3.0)
    a = kernels.swiglu(gu)
    g, u = gu.double()[:, 0::2], gu.double()[:, 1::2]
    torch.testing.assert_close(a.double(), P.silu(g) * u, **tol(dt))


def paged(seq_lens, nkv, hd, dt, n_pages=40, seed=0, shuffle=True):
    """Random keys/values for sequences of the given lengths, scattered over shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g).tolist() if shuffle else list(range(n_pages))
    max_pages = max((n + 63) // 64 for n in seq_lens) + 1
    table = torch.zeros(len(seq_lens) + 2, max_pages, dtype=torch.int32)
    k_pages = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=dt)
    v_pages = torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=dt)
    ks, vs = [], []
    for s, n in enumerate(seq_lens):
        k = torch.randn(n, nkv, hd, generator=g).to(dt)
        v = torch.randn(n, nkv, hd, generator=g).to(dt)
        ks.append(k); vs.append(v)
        for p in range((n + 63) // 64):
            page = order.pop()
            table[s + 1, p] = page                      # sequence s lives in slot s + 1
            m = min(64, n - p * 64)
            k_pages[page, :, :m] = k[p * 64:p * 64 + m].transpose(0, 1)
            v_pages[page, :, :m] = v[p * 64:p * 64 + m].transpose(0, 1)
    return ks, vs, k_pages.to(DEV), v_pages.to(DEV), table.to(DEV)


def attention_reference(q, k, v, pos, scale, window):
    """q [nh, hd] at absolute position pos over k/v [n, nkv, hd] (float64)."""
    nh, hd = q.shape
    nkv = k.shape[1]
    lo = 0 if not window else max(0, pos - window + 1)
    out = torch.zeros(nh, hd, dtype=torch.float64)
    for h in range(nh):
        kh = h // (nh // nkv)
        s = (k[lo:pos + 1, kh].double() @ q[h].double()) * scale
        w = torch.softmax(s, dim=0)
        out[h] = w @ v[lo:pos + 1, kh].double()
    return out


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, None), (6, 1, 48, None), (8, 8, 80, 70),
                                              (14, 2, 64, None), (28, 4, 128, 200), (2, 2, 256, None)])
def test_attention_generic(dt, nh, nkv, hd, window):
    """New tokens of three sequences (a whole prompt, an appended chunk, one decoded token)."""
    from rocmforge_b200 import kernels
    lens = [150, 333, 65]
    new = [150, 20, 1]
    ks, vs, k_pages, v_pages, table = paged(lens, nkv, hd, dt, seed=nh)
    g = torch.Generator().manual_seed(1)
    T = sum(new)
    q = torch.randn(T, nh * hd, generator=g).to(dt)
    tok_seq = torch.tensor(sum(([i] * n for i, n in enumerate(new)), []), dtype=torch.int32)
    tok_pos = torch.tensor(sum((list(range(L - n, L)) for L, n in zip(lens, new)), []), dtype=torch.int32)
    seq_slot = torch.tensor([1, 2, 3], dtype=torch.int32)
    scale = 1.0 / math.sqrt(hd)
    out = kernels.attention_generic(q.to(DEV), nh, nkv, hd, k_pages, v_pages, tok_seq.to(DEV), tok_pos.to(DEV),
                                    seq_slot.to(DEV), table, scale, window)
    assert torch.isfinite(out).all(), "a page that holds no key of the sequence was read"
    for t in range(T):
        s = int(tok_seq[t])
        ref = attention_reference(q[t].view(nh, hd), ks[s], vs[s], int(tok_pos[t]), scale, window)
        torch.testing.assert_close(out[t].cpu().double().view(nh, hd), ref, **tol(dt))


@pytest.mark.parametrize("dt", DTS)
def test_attention_finds_one_far_key_and_the_window_edge(dt):
    """Random weights hide a key that is never read: make one far key (and the two keys at the
    window's edge) stand out by a large, aligned score, and check whose value comes out."""
    from rocmforge_b200 import kernels
    nh = nkv = 1
    hd, n = 32, 700
    ks, vs, k_pages, v_pages, table = paged([n], nkv, hd, dt, n_pages=16, seed=3)
    q = torch.zeros(1, hd); q[0, 0] = 8.0
    args = (torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([n - 1], dtype=torch.int32, device=DEV),
            torch.tensor([1], dtype=torch.int32, device=DEV), table)

    def run(target, window):
        kp = k_pages.clone()
        page = int(table[1, target // 64])
        kp[page, 0, target % 64] = 0
        kp[page, 0, target % 64, 0] = 40.0              # score 8 * 40 / sqrt(32): dwarfs every other key
        return kernels.attention_generic(q.to(dt).to(DEV), nh, nkv, hd, kp, v_pages, *args,
                                         1.0 / math.sqrt(hd), window)[0].float().cpu()

    for target in (0, 3, 63, 64, 320, 698):
        torch.testing.assert_close(run(target, None), vs[0][target, 0].float(), atol=1e-3, rtol=1e-3)
    W = 100                                             # the query at 699 sees keys 600..699
    torch.testing.assert_close(run(600, W), vs[0][600, 0].float(), atol=1e-3, rtol=1e-3)
    out = run(599, W)                                   # one position outside: must be ignored
    assert (out - vs[0][599, 0].float()).abs().max() > 0.1
    ref = attention_reference(q.to(dt).view(1, hd), ks[0], vs[0], n - 1, 1.0 / math.sqrt(hd), W)
    torch.testing.assert_close(out.double().view(1, hd), ref, **tol(dt))


def plain_rotation(x, pos, inv_freq, rot_dim, interleaved):
    """x [T, heads, hd] turned as maeddesg/ROCmForge src/cpu/ops.rs:69-98 does it: pair i of the first rot_dim
    elements by the 32-bit angle pos * inv_freq[i]; pairs are (i, i + rot_dim/2) (neox) or (2i, 2i+1)."""
    ang = (pos.to(torch.float32)[:, None] * inv_freq.float()[None, :]).double()
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:rot_dim:2], x[..., 1:rot_dim:2]
        out[..., 0:rot_dim:2], out[..., 1:rot_dim:2] = a * c - b * s, a * s + b * c
    else:
        h = rot_dim // 2
        a, b = x[..., :h], x[..., h:rot_dim]
        out[..., :h], out[..., h:rot_dim] = a * c - b * s, a * s + b * c
    return out


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("hd,rot_dim,interleaved", [(64, 64, True), (64, 32, False), (48, 16, True), (128, 0, False), (32, 2, False)])
def test_rope_kv_write_partial_and_interleaved_rotations(dt, hd, rot_dim, interleaved):
    """Only the first rot_dim elements of a head turn, as split or as neighbouring pairs; none at all with rot_dim 0.
    Through both entries of the kernel: rows of one tensor (one token and 70) and partial sums plus bias."""
    from rocmforge_b200 import kernels
    nh, nkv = 6, 2
    width = (nh + 2 * nkv) * hd
    inv = (1.0 / (1e4 ** (torch.arange(rot_dim // 2, dtype=torch.float64) * 2 / max(rot_dim, 1)))).float().to(DEV) if rot_dim else None
    for T in (1, 70):
        pos = torch.randint(0, 3000, (T,), generator=torch.Generator().manual_seed(T)).to(torch.int32)
        table = torch.arange(64, dtype=torch.int32).view(1, 64).to(DEV)
        seq, slot = torch.zeros(T, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV)
        parts = rnd(3, T, width, seed=9)
        bias = rnd(width, seed=10)
        total = parts.double().sum(0).cpu() + bias.double().cpu()
        for source in ("rows", "partials"):
            k_pages = torch.zeros(64, nkv, 64, hd, dtype=dt, device=DEV)
            v_pages = torch.zeros_like(k_pages)
            if source == "rows":
                qkv = total.to(dt).to(DEV)
                x = qkv.double().cpu()
                q = kernels.rope_kv_write(qkv, nh, nkv, hd, inv, seq, pos.to(DEV), slot, table, k_pages, v_pages,
                                          rot_dim=rot_dim, interleaved=interleaved)[:, :nh * hd]
            else:
                x = total
                q = kernels.rope_kv_write(parts, nh, nkv, hd, inv, seq, pos.to(DEV), slot, table, k_pages, v_pages, bias=bias,
                                          compute_dtype=dt, rot_dim=rot_dim, interleaved=interleaved)
            turn = (lambda t: plain_rotation(t, pos, inv.cpu(), rot_dim, interleaved)) if rot_dim else (lambda t: t)
            q_ref = turn(x[:, :nh * hd].reshape(T, nh, hd))
            k_ref = turn(x[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd))
            v_ref = x[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
            torch.testing.assert_close(q.double().cpu().view(T, nh, hd), q_ref, **tol(dt))
            # a later token at the same position overwrites an earlier one: compare the last writer of each position
            last = {int(p_): i for i, p_ in enumerate(pos.tolist())}
            for p_, i in last.items():
                torch.testing.assert_close(k_pages[p_ // 64, :, p_ % 64].double().cpu(), k_ref[i], **tol(dt))
                torch.testing.assert_close(v_pages[p_ // 64, :, p_ % 64].double().cpu(), v_ref[i], **tol(dt))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (3, 1, 48), (28, 4, 128)])
def test_rope_kv_write(dt, nh, nkv, hd):
    from rocmforge_b200 import kernels
    from rocmforge_b200.parts import NeoxRope
    theta = 1e6
    rope = NeoxRope(hd, theta); rope.prepare(DEV)
    pos = torch.tensor([0, 1, 63, 64, 65, 4000, 7], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 0, 0, 1, 2], dtype=torch.int32)
    T = len(pos)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dt=dt, seed=5)
    before = qkv.clone()
    n_pages, max_pages = 80, 64
    table = torch.zeros(4, max_pages, dtype=torch.int32)
    table[1, 0], table[1, 1], table[2, 4000 // 64], table[3, 0] = 7, 3, 11, 5
    k_pages = torch.zeros(n_pages, nkv, 64, hd, dtype=dt, device=DEV)
    v_pages = torch.zeros_like(k_pages)
    kernels.rope_kv_write(qkv, nh, nkv, hd, rope.inv_freq, seq.to(DEV), pos.to(DEV),
                          torch.tensor([1, 2, 3], dtype=torch.int32, device=DEV), table.to(DEV), k_pages, v_pages)
    b = before.double().cpu()
    q_ref = P.rope_neox(b[:, :nh * hd].view(T, nh, hd), pos, theta)
    k_ref = P.rope_neox(b[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd), pos, theta)
    v_ref = b[:, (nh + nkv) * hd:].view(T, nkv, hd)
    t = tol(dt)
    torch.testing.assert_close(qkv[:, :nh * hd].double().cpu().view(T, nh, hd), q_ref, **t)
    assert torch.equal(qkv[:, nh * hd:], before[:, nh * hd:])          # k and v columns stay as they were
    where = [(7, 0), (7, 1), (7, 63), (3, 0), (3, 1), (11, 4000 % 64), (5, 7)]
    for i, (page, off) in enumerate(where):
        torch.testing.assert_close(k_pages[page, :, off].double().cpu(), k_ref[i], **t)
        torch.testing.assert_close(v_pages[page, :, off].double().cpu(), v_ref[i], atol=0, rtol=0)
    assert int((k_pages.float().abs().sum(dim=(1, 3)) > 0).sum()) == T    # nothing else was written
    # a layer that reads another layer's cache rotates q and writes nothing
    qkv2 = before.clone()
    k2 = torch.zeros_like(k_pages)
    kernels.rope_kv_write(qkv2, nh, nkv, hd, rope.inv_freq, seq.to(DEV), pos.to(DEV),
                          torch.tensor([1, 2, 3], dtype=torch.int32, device=DEV), table.to(DEV), k2, k2,
                          write_kv=False)
    assert torch.equal(qkv2, qkv) and float(k2.abs().sum()) == 0


@pytest.mark.parametrize("nh,nkv,hd,window", [(28, 4, 128, None), (14, 2, 64, None), (4, 4, 64, 300), (8, 1, 128, None),
                                              (3, 3, 256, None), (12, 4, 128, 1000), (8, 2, 64, 64), (5, 1, 64, 130)])
def test_attention_decode(nh, nkv, hd, window):
    """One new token per sequence over contexts that end inside, at and beyond chunk borders."""
    from rocmforge_b200 import kernels
    dt = torch.bfloat16
    lens = [1, 255, 256, 257, 700, 1500, 64]
    B = len(lens)
    ks, vs, k_pages, v_pages, table = paged(lens, nkv, hd, dt, n_pages=64, seed=nh + hd)
    g = torch.Generator().manual_seed(2)
    q = torch.randn(B, nh * hd, generator=g).to(dt)
    tok_seq = torch.arange(B, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seq_slot = torch.arange(1, B + 1, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    refs = [attention_reference(q[b].view(nh, hd), ks[b], vs[b], lens[b] - 1, scale, window) for b in range(B)]
    for max_chunks in (12, 32):                            # exactly enough, and a replayed graph's fixed shape
        n_o, n_ml, n_c = kernels.attention_decode_scratch(B, nh, nkv, hd, max_chunks)
        part_o = torch.full((n_o,), float("nan"), device=DEV)
        part_ml = torch.full((n_ml,), float("nan"), device=DEV)
        counters = torch.zeros(n_c, dtype=torch.int32, device=DEV)
        for rep in range(2):                               # the second launch finds the counters as the first left them
            out = kernels.attention_decode(q.to(DEV), nh, nkv, hd, k_pages, v_pages, tok_seq, tok_pos, seq_slot,
                                           table, scale, window, max_chunks, part_o, part_ml, counters)
            assert torch.isfinite(out.float()).all()
            assert int(counters.abs().sum()) == 0
            for b in range(B):
                torch.testing.assert_close(out[b].cpu().double().view(nh, hd), refs[b], atol=2e-2, rtol=2e-2)
    gen = kernels.attention_generic(q.to(DEV), nh, nkv, hd, k_pages, v_pages, tok_seq, tok_pos, seq_slot, table,
                                    scale, window)
    torch.testing.assert_close(out.float(), gen.float(), atol=2e-2, rtol=2e-2)
    # the clustered kernel: every cluster size and both CTA widths, the same answers
    for splits, warps in ((1, 4), (1, 8), (2, 8), (4, 4), (8, 8), (16, 8)):
        out = kernels.attention_decode_warps(q.to(DEV), nh, nkv, hd, k_pages, v_pages, tok_seq, tok_pos, seq_slot,
                                             table, scale, window, splits=splits, warps=warps)
        assert torch.isfinite(out.float()).all()
        for b in range(B):
            torch.testing.assert_close(out[b].cpu().double().view(nh, hd), refs[b], atol=2e-2, rtol=2e-2)
    assert kernels.decode_splits(1, 4) == 8 and kernels.decode_splits(8, 4) == 4 and kernels.decode_splits(64, 4) == 1
    assert kernels.decode_splits(1, 4, longest=100) == 2 and kernels.decode_splits(1, 4, 4096, window=128) == 2
    assert kernels.decode_splits(1, 4, longest=4096) == 16 and kernels.decode_splits(2, 4, longest=4096) == 8
    assert kernels.decode_pages(1 << 20, 1024) == 17            # a window bounds the pages whatever the length


def test_attention_decode_finds_far_keys_and_the_window_edge():
    from rocmforge_b200 import kernels
    dt, nh, nkv, hd, n = torch.bfloat16, 2, 1, 64, 900
    ks, vs, k_pages, v_pages, table = paged([n], nkv, hd, dt, n_pages=20, seed=5)
    q = torch.zeros(1, nh * hd); q[0, 0] = 8.0; q[0, hd + 1] = 8.0      # head 0 looks along dim 0, head 1 along dim 1
    zero = torch.zeros(1, dtype=torch.int32, device=DEV)
    n_o, n_ml, n_c = kernels.attention_decode_scratch(1, nh, nkv, hd, 8)
    scratch = (torch.zeros(n_o, device=DEV), torch.zeros(n_ml, device=DEV), torch.zeros(n_c, dtype=torch.int32, device=DEV))

    which = {"kernel": "chunked"}

    def run(t0, t1, window):
        kp = k_pages.clone()
        for dim, t in ((0, t0), (1, t1)):
            page = int(table[1, t // 64])
            kp[page, 0, t % 64, dim] = 60.0
        args = (q.to(dt).to(DEV), nh, nkv, hd, kp, v_pages, zero, torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                torch.tensor([1], dtype=torch.int32, device=DEV), table, 1.0 / math.sqrt(hd), window)
        if which["kernel"] == "chunked":
            return kernels.attention_decode(*args, 8, *scratch)[0].float().cpu().view(nh, hd)
        return kernels.attention_decode_warps(*args, splits=splits, warps=warps)[0].float().cpu().view(nh, hd)

    splits = warps = 0
    check_far_keys(run, vs)
    which["kernel"] = "clustered"
    for splits, warps in ((4, 8), (1, 4), (8, 4)):
        check_far_keys(run, vs)


def check_far_keys(run, vs):
    for t0, t1 in ((0, 899), (127, 128), (511, 512), (63, 64), (700, 3), (895, 896)):
        out = run(t0, t1, None)
        torch.testing.assert_close(out[0], vs[0][t0, 0].float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(out[1], vs[0][t1, 0].float(), atol=2e-2, rtol=2e-2)
    out = run(500, 499, 400)                             # the query at 899 sees 500..899: 500 is in, 499 is out
    torch.testing.assert_close(out[0], vs[0][500, 0].float(), atol=2e-2, rtol=2e-2)
    assert (out[1] - vs[0][499, 0].float()).abs().max() > 0.1


@pytest.mark.parametrize("nh,nkv,hd,window", [(28, 4, 128, None), (14, 2, 64, None), (4, 4, 64, 100), (6, 1, 128, 70),
                                              (2, 2, 128, 64), (3, 1, 64, 1)])
@pytest.mark.parametrize("kernel", ["mma_sync", "tcgen05"])
def test_attention_prefill(nh, nkv, hd, window, kernel):
    """Tiled attention: a whole prompt, a chunk appended to a context, tiny and page-straddling pieces."""
    from rocmforge_b200 import kernels
    tile, run = (64, kernels.attention_prefill) if kernel == "mma_sync" else (128, kernels.attention_prefill_tc)
    dt = torch.bfloat16
    lens = [300, 333, 65, 1, 64, 130]
    new = [300, 50, 65, 1, 3, 129]
    ks, vs, k_pages, v_pages, table = paged(lens, nkv, hd, dt, n_pages=48, seed=nh * hd)
    g = torch.Generator().manual_seed(3)
    T = sum(new)
    q = torch.randn(T, nh * hd, generator=g).to(dt)
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    tiles = [(i, q0) for i, n in enumerate(new) for q0 in range(0, n, tile)]
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    out = run(q.to(DEV), nh, nkv, hd, k_pages, v_pages, dev(tiles).view(-1),
                                    dev(list(range(1, len(lens) + 1))), dev([L - n for L, n in zip(lens, new)]),
                                    dev(new), dev(cu), table, scale, window)
    assert torch.isfinite(out.float()).all()
    t = 0
    for s, (L, n) in enumerate(zip(lens, new)):
        for r in range(n):
            ref = attention_reference(q[t].view(nh, hd), ks[s], vs[s], L - n + r, scale, window)
            torch.testing.assert_close(out[t].cpu().double().view(nh, hd), ref, atol=2e-2, rtol=2e-2)
            t += 1


def test_attention_prefill_gives_the_same_bits_launch_after_launch():
    """Many short launches of the tcgen05 kernel over ragged sequences of one to six pages: every launch the bits of the
    first one and no wait that ran out.  The kernel's warps hand work to each other through barriers that are
    told apart by one parity bit; a barrier that completes two phases between two looks of a waiter shows here as a CTA
    that stands still until its wait's limit, or as other bits."""
    from rocmforge_b200 import kernels
    from rocmforge_b200.kernels import tensor_core as tc
    dt, nh, nkv, hd = torch.bfloat16, 14, 2, 64
    g = torch.Generator().manual_seed(21)
    lens = torch.randint(1, 400, (48,), generator=g).tolist()
    ks, vs, k_pages, v_pages, table = paged(lens, nkv, hd, dt, n_pages=sum((n + 63) // 64 for n in lens) + 2, seed=8)
    T = sum(lens)
    q = torch.randn(T, nh * hd, generator=g).to(dt).to(DEV)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    tiles = [(i, q0) for i, n in enumerate(lens) for q0 in range(0, n, 128)]
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    args = (dev(tiles).view(-1), dev(list(range(1, len(lens) + 1))), dev([0] * len(lens)), dev(lens), dev(cu), table,
            1.0 / math.sqrt(hd), None)
    first = kernels.attention_prefill_tc(q, nh, nkv, hd, k_pages, v_pages, *args).clone()
    t = 0
    for s, n in enumerate(lens[:6]):
        ref = attention_reference(q[t + n - 1].cpu().view(nh, hd), ks[s], vs[s], n - 1, 1.0 / math.sqrt(hd), None)
        torch.testing.assert_close(first[t + n - 1].cpu().double().view(nh, hd), ref, atol=2e-2, rtol=2e-2)
        t += n
    # as in a prompt step, the product that reads the result is launched behind every attention launch: it starts while
    # the attention kernel still runs, and its waiting warps take issue slots from the attention's warps
    w_o = rnd(nh * hd, nh * hd, dt=dt, seed=3) * 0.05
    h = torch.zeros(T, nh * hd, device=DEV)
    outs = []
    for rep in range(200):
        out = kernels.attention_prefill_tc(q, nh, nkv, hd, k_pages, v_pages, *args)
        tc.gemm_tc(out, w_o, mode=tc.RESIDUAL, out=h)
        outs.append(out)
        if len(outs) == 50:                              # compared in batches, so that the launches follow each other closely
            differ = sum(int(not torch.equal(o, first)) for o in outs)
            assert differ == 0, f"{differ} of 50 launches gave other bits than the first"
            outs = []
    tc.check_status(DEV)


@pytest.mark.parametrize("kernel", ["mma_sync", "tcgen05"])
def test_attention_prefill_finds_far_keys_and_the_window_edge(kernel):
    from rocmforge_b200 import kernels
    fn = kernels.attention_prefill if kernel == "mma_sync" else kernels.attention_prefill_tc
    dt, nh, nkv, hd, n = torch.bfloat16, 1, 1, 64, 700
    ks, vs, k_pages, v_pages, table = paged([n], nkv, hd, dt, n_pages=16, seed=9)
    # the last two rows are the queries; both look along dim 0
    q = torch.zeros(2, hd); q[:, 0] = 8.0
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)

    def run(target, window):
        kp = k_pages.clone()
        page = int(table[1, target // 64])
        kp[page, 0, target % 64] = 0
        kp[page, 0, target % 64, 0] = 60.0
        return fn(q.to(dt).to(DEV), nh, nkv, hd, kp, v_pages, dev([0, 0]), dev([1]), dev([n - 2]),
                  dev([2]), dev([0, 2]), table, 1.0 / math.sqrt(hd), window).float().cpu()

    for target in (0, 63, 64, 320, 697):
        out = run(target, None)
        for row in range(2):
            torch.testing.assert_close(out[row], vs[0][target, 0].float(), atol=2e-2, rtol=2e-2)
    out = run(599, 100)            # rows at 698 and 699 with a window of 100: 599 is inside for the first row only
    torch.testing.assert_close(out[0], vs[0][599, 0].float(), atol=2e-2, rtol=2e-2)
    assert (out[1] - vs[0][599, 0].float()).abs().max() > 0.1
    out = run(699, None)           # the last key belongs to the second row alone (causal)
    torch.testing.assert_close(out[1], vs[0][699, 0].float(), atol=2e-2, rtol=2e-2)
    assert (out[0] - vs[0][699, 0].float()).abs().max() > 0.1


@pytest.mark.parametrize("nh,nkv,hd,S", [(6, 2, 32, 3), (28, 4, 128, 8), (14, 2, 64, 19), (5, 1, 24, 9), (3, 1, 20, 4),
                                         (40, 8, 128, 11)])
def test_rope_kv_write_from_partial_sums(nh, nkv, hd, S):
    """The rotation kernel adds the 32-bit partial sums of a K-split product and the bias itself: up to eight splits in
    one round of loads, more in several; head sizes that are and are not multiples of 8."""
    from rocmforge_b200 import kernels
    from rocmforge_b200.parts import NeoxRope
    T = 5
    width = (nh + 2 * nkv) * hd
    rope = NeoxRope(hd, 1e4); rope.prepare(DEV)
    parts = rnd(S, T, width, seed=1)
    bias = rnd(width, seed=2)
    pos = torch.tensor([0, 5, 64, 130, 9], dtype=torch.int32, device=DEV)
    seq = torch.arange(T, dtype=torch.int32, device=DEV)
    slots = torch.arange(T, dtype=torch.int32, device=DEV)
    table = (torch.arange(T * 4, dtype=torch.int32).view(T, 4)).to(DEV)
    total = (parts.sum(0) + bias)
    for dt in DTS:
        kp = torch.zeros(T * 4, nkv, 64, hd, dtype=dt, device=DEV)
        vp = torch.zeros_like(kp)
        q = kernels.rope_kv_write(parts, nh, nkv, hd, rope.inv_freq, seq, pos, slots, table, kp, vp, bias=bias,
                                  compute_dtype=dt)
        kp2, vp2 = torch.zeros_like(kp), torch.zeros_like(vp)
        whole = total.to(dt).clone()
        q2 = kernels.rope_kv_write(whole, nh, nkv, hd, rope.inv_freq, seq, pos, slots, table, kp2, vp2)
        t = dict(atol=1e-5, rtol=1e-5) if dt == torch.float32 else dict(atol=4e-2, rtol=2e-2)
        torch.testing.assert_close(q.float(), q2[:, :nh * hd].float(), **t)
        torch.testing.assert_close(kp.float(), kp2.float(), **t)
        torch.testing.assert_close(vp.float(), vp2.float(), **t)
        assert tuple(q.shape) == (T, nh * hd) and q.dtype == dt


def test_argmax_ties_and_sizes():
    from rocmforge_b200 import kernels
    x = rnd(5, 152064, seed=9)
    x[0, 17] = x[0, 150000] = 50.0
    x[1, 0] = 60.0
    x[2, 152063] = 60.0
    x[3] = 0.0
    got = kernels.argmax(x).cpu().tolist()
    assert got[:4] == [150000, 0, 152063, 152063]            # equal maxima: the highest index
    assert got[4] == S.greedy(x[4].cpu())
    y = rnd(3, 300, seed=1)
    assert kernels.argmax(y).cpu().tolist() == [S.greedy(r) for r in y.cpu()]
    # every split of a row over CTAs (16 down to 1 with the number of rows), winners planted in every part of the row
    for rows, V in ((1, 152064), (20, 152064), (64, 151936), (300, 40000), (3, 9000), (7, 8191)):
        z = rnd(rows, V, seed=rows)
        want = []
        for r in range(rows):
            at = (r * 7919 + 13) * 104729 % V
            z[r, at] = 40.0
            if r % 3 == 0:
                z[r, min(V - 1, at + 4097)] = 40.0               # an equal maximum further on, often in another CTA's part
                at = max(at, min(V - 1, at + 4097))
            want.append(at)
        z[0, 5] = float("nan")                                   # a NaN never wins
        assert kernels.argmax(z).cpu().tolist() == want, (rows, V)
    wide = rnd(6, 1003, seed=3)                                   # rows that start off 16-byte borders
    view = wide[:, 1:1002]
    assert kernels.argmax(view).cpu().tolist() == [S.greedy(r) for r in view.cpu()]
    nans = torch.full((2, 5000), float("nan"), device=DEV)
    nans[1, 4321] = -3.0
    assert kernels.argmax(nans).cpu().tolist() == [0, 4321]


@pytest.fixture(params=[True, False], ids=["slice in shared memory", "row in global memory"])
def cached(request):
    """Both samplers (they must give the same token; the second also serves vocabularies beyond the first one's reach)."""
    from rocmforge_b200 import kernels
    kernels.set_sample_cached(request.param)
    yield request.param
    kernels.set_sample_cached(True)


@pytest.mark.parametrize("V", [300, 5000, 152064, 200000, 320000])
def test_sample_kernel_follows_the_plain_sampler(V, cached):
    from rocmforge_b200 import kernels
    from rocmforge_b200.sampling import as_int64, draw_seed
    R = 24 if V < 100000 else 12
    logits = rnd(R, V, seed=V, scale=2.5)
    logits[:, 5] = logits[:, 77]                              # equal logits somewhere in every row
    logits[3, :] = 0.25                                       # a row of equal logits but one (all equal
    logits[3, 0] = 1.0                                        # would put top_p * V exactly on a boundary)
    cpu = logits.cpu()
    for temperature, top_p, top_k in ((0.8, 1.0, 0), (0.8, 0.9, 0), (1.0, 0.5, 0), (1.5, 1.0, 40),
                                      (0.7, 0.8, 10), (1.0, 0.95, 1), (1e-7, 1.0, 0), (1.0, 0.0, 0)):
        seeds = [draw_seed(1234, r, 3) for r in range(R)]
        got = kernels.sample(logits, temperature, top_p, top_k,
                             torch.tensor([as_int64(s) for s in seeds], dtype=torch.int64, device=DEV)).cpu().tolist()
        want = [S.sample(cpu[r], temperature, top_p, top_k, seeds[r]) for r in range(R)]
        assert got == want, f"temperature={temperature} top_p={top_p} top_k={top_k}"
    # the draw counter advances the seed on the device
    base = torch.tensor([as_int64(draw_seed(99, r, 0)) for r in range(R)], dtype=torch.int64, device=DEV)
    counter = torch.tensor([5], dtype=torch.int32, device=DEV)
    got = kernels.sample(logits, 0.9, 0.9, 0, base, draw_counter=counter).cpu().tolist()
    assert got == [S.sample(cpu[r], 0.9, 0.9, 0, draw_seed(99, r, 5)) for r in range(R)]


@pytest.mark.parametrize("R", [1, 3, 8, 24, 60, 100])
def test_sample_kernel_with_every_cluster_size(R, cached):
    """The CTAs per row go with the number of rows (16, 8, 4, 2, 1); small vocabularies leave some CTAs without an element."""
    from rocmforge_b200 import kernels
    from rocmforge_b200.sampling import as_int64, draw_seed
    for V in (5, 97, 3001):
        logits = rnd(R, V, seed=R + V, scale=2.0)
        logits[:, V // 2] = logits[:, 0]
        cpu = logits.cpu()
        for temperature, top_p, top_k in ((0.8, 0.9, 0), (1.0, 1.0, 3), (1.3, 0.6, 0)):
            seeds = [draw_seed(77, r, 1) for r in range(R)]
            got = kernels.sample(logits, temperature, top_p, top_k,
                                 torch.tensor([as_int64(s) for s in seeds], dtype=torch.int64, device=DEV)).cpu().tolist()
            assert got == [S.sample(cpu[r], temperature, top_p, top_k, seeds[r]) for r in range(R)], (R, V, temperature, top_p, top_k)


def test_both_samplers_pick_the_same_tokens():
    """The sampler with the slice in shared memory against the one that walks global memory, on rows of every kind:
    nearly flat (a random model's logits), peaked, with masked-out tokens, all equal, two values only."""
    from rocmforge_b200 import kernels
    R, V = 40, 152064
    rows = [rnd(R, V, seed=1, scale=0.3), rnd(R, V, seed=2, scale=6.0)]
    masked = rnd(R, V, seed=3, scale=2.0)
    masked[:, ::3] = float("-inf")
    masked[5, :] = float("-inf")
    masked[5, 777] = 0.5
    rows.append(masked)
    flat = torch.zeros(R, V, device=DEV)
    flat[1::2, 1000:2000] = 1.0
    rows.append(flat)
    quant = (rnd(R, V, seed=4, scale=2.0) * 4).round() / 4               # many ties at every level
    rows.append(quant)
    seeds = torch.arange(R, dtype=torch.int64, device=DEV) * 7919 + 17
    try:
        for logits in rows:
            for temperature, top_p, top_k in ((1.0, 0.9, 0), (0.7, 1.0, 0), (1.3, 0.3, 0), (1.0, 0.95, 50), (1.0, 1.0, 5)):
                for draw in range(3):
                    counter = torch.tensor([draw * 1000003], dtype=torch.int32, device=DEV)
                    kernels.set_sample_cached(True)
                    a = kernels.sample(logits, temperature, top_p, top_k, seeds, draw_counter=counter).clone()
                    kernels.set_sample_cached(False)
                    b = kernels.sample(logits, temperature, top_p, top_k, seeds, draw_counter=counter)
                    assert torch.equal(a, b), (temperature, top_p, top_k, draw, (a != b).nonzero().flatten().tolist())
    finally:
        kernels.set_sample_cached(True)


def test_kernels_refuse_what_they_cannot_do():
    from rocmforge_b200 import kernels
    from rocmforge_b200.kernels import KernelError
    with pytest.raises(KernelError):
        kernels.embed(torch.zeros(4, 4), torch.zeros(2, dtype=torch.int32))            # CPU tensors
    with pytest.raises(KernelError):
        kernels.gemm_simt(rnd(2, 8), rnd(3, 9))                                          # inner sizes differ
    with pytest.raises(KernelError):
        kernels.gemm_simt(rnd(2, 8, dt=torch.float16), rnd(3, 8, dt=torch.float16))      # dtype without a kernel
    with pytest.raises(KernelError):
        kernels.add_rmsnorm(rnd(2, 60000), rnd(60000), 1e-6, torch.float32)             # row larger than shared memory
    with pytest.raises(KernelError):
        kernels.swiglu(rnd(2, 7))
