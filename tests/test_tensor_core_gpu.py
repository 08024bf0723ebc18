"""The tcgen05 matrix products alone, against float64 references (needs a GPU)."""
import pytest
import torch

from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, scale=1.0, dt=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dt).to(DEV)


def close(got, ref, what=""):
    """bfloat16 operands, 32-bit sums: within 1 % of the largest value for bf16 outputs, 1e-3 for f32 ones."""
    scale = float(ref.abs().max())
    rel = 1e-2 if got.dtype == torch.bfloat16 else 1e-4
    err = float((got.double() - ref).abs().max())
    assert err <= rel * scale, f"{what}: largest difference {err:.4g}, allowed {rel * scale:.4g}"


SHAPES = [(1, 128, 64), (5, 48, 72), (128, 256, 128), (130, 200, 264), (300, 520, 1000), (2048, 4608, 3584),
          (77, 3584, 18944), (257, 1000, 3584)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_tokens_as_rows(M, N, K):
    from rocmforge_b200.kernels import tensor_core as tc
    x, w, b = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=0.05), rnd(N, seed=3, dt=torch.float32)
    ref = x.double() @ w.double().t()
    close(tc.gemm_tc(x, w), ref, "store")
    close(tc.gemm_tc(x, w, b, mode=tc.F32), ref + b.double(), "f32 + bias")
    close(tc.gemm_tc(x, w, b.bfloat16()), ref + b.bfloat16().double(), "bf16 bias")
    acc = rnd(M, N, seed=4, dt=torch.float32)
    want = acc.double() + ref
    tc.gemm_tc(x, w, mode=tc.RESIDUAL, out=acc)
    close(acc, want, "residual")
    if N % 2 == 0:
        g, u = ref[:, 0::2], ref[:, 1::2]
        close(tc.gemm_tc(x, w, mode=tc.SWIGLU), P.silu(g) * u, "swiglu")
    tc.check_status(DEV)


@pytest.mark.parametrize("cluster", [2, 4, "pair"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (300, 520, 1000), (2048, 4608, 3584), (1100, 3584, 18944),
                                   (257, 1000, 3584), (640, 37888, 3584), (65, 3584, 3584), (128, 4608, 3584),
                                   (200, 3584, 18944)])
def test_clustered_persistent_kernel(M, N, K, cluster):
    from rocmforge_b200.kernels import tensor_core as tc
    if not tc.cluster_available():
        pytest.skip("the clustered module is not part of this checkout")
    # "pair": the two CTAs of a cluster as one MMA unit; 2 and 4: CTAs that multicast weight tiles to each other
    was = tc.cluster_pair()
    tc.set_cluster_pair(cluster == "pair")
    try:
        clustered_cases(tc, M, N, K, 2 if cluster == "pair" else cluster)
    finally:
        tc.set_cluster_pair(was)


def clustered_cases(tc, M, N, K, cluster):
    x, w, b = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=0.05), rnd(N, seed=3, dt=torch.float32)
    ref = x.double() @ w.double().t()
    close(tc.gemm_tc(x, w, cluster=cluster), ref, "store")
    close(tc.gemm_tc(x, w, b, mode=tc.F32, cluster=cluster), ref + b.double(), "f32 + bias")
    acc = rnd(M, N, seed=4, dt=torch.float32)
    want = acc.double() + ref
    tc.gemm_tc(x, w, mode=tc.RESIDUAL, out=acc, cluster=cluster)
    close(acc, want, "residual")
    close(tc.gemm_tc(x, w, mode=tc.SWIGLU, cluster=cluster), P.silu(ref[:, 0::2]) * ref[:, 1::2], "swiglu")
    assert torch.equal(tc.gemm_tc(x, w, cluster=cluster), tc.gemm_tc(x, w, cluster=0)), "both kernels sum in the same order"
    for parts in (2, 3, 5):
        kb = (K + 63) // 64
        if (parts - 1) * ((kb + parts - 1) // parts) >= kb:      # a part would be empty: the kernel refuses
            continue
        # K cut in parts whose sums are added one after the other: the same sums in one fixed order, launch after launch
        runs = []
        for rep in range(2):
            acc = rnd(M, N, seed=4, dt=torch.float32)
            tc.gemm_tc(x, w, b, mode=tc.RESIDUAL, out=acc, cluster=cluster, parts=parts)
            close(acc, want + b.double(), f"{parts} K parts")
            runs.append(acc)
        assert torch.equal(runs[0], runs[1]), "the order of the parts is fixed"
        assert int(tc.part_flags(DEV).abs().sum()) == 0, "the counters are left zeroed"
    tc.check_status(DEV)


@pytest.mark.parametrize("M", [1, 3, 8, 16, 17, 33, 64, 65, 100, 128])
@pytest.mark.parametrize("N,K", [(128, 64), (200, 136), (3584, 3584), (1000, 18944), (4608, 3584)])
def test_weights_as_rows(M, N, K):
    from rocmforge_b200.kernels import tensor_core as tc
    x, w, b = rnd(M, K, seed=5), rnd(N, K, seed=6, scale=0.05), rnd(N, seed=7, dt=torch.float32)
    ref = x.double() @ w.double().t()
    close(tc.gemm_tc_skinny(x, w), ref, "store")
    close(tc.gemm_tc_skinny(x, w, b, mode=tc.F32), ref + b.double(), "f32 + bias")
    acc = rnd(M, N, seed=8, dt=torch.float32)
    want = acc.double() + ref
    tc.gemm_tc_skinny(x, w, mode=tc.RESIDUAL, out=acc)
    close(acc, want, "residual")
    if N % 2 == 0:
        close(tc.gemm_tc_skinny(x, w, mode=tc.SWIGLU), P.silu(ref[:, 0::2]) * ref[:, 1::2], "swiglu")
    splits = tc.split_k_for(N, K)
    for s in {1, splits, min(3, (K + 63) // 64)}:
        parts = tc.gemm_tc_skinny(x, w, mode=tc.PARTIAL, splits=s)
        assert tuple(parts.shape) == (s, M, N)
        close(parts.double().sum(0).float(), ref, f"{s} partial sums")
    # a token's result does not depend on the others in the batch
    if M > 1:
        alone = tc.gemm_tc_skinny(x[M - 1:M], w, mode=tc.F32)
        assert torch.equal(alone, tc.gemm_tc_skinny(x, w, mode=tc.F32)[M - 1:M])
    tc.check_status(DEV)


@pytest.mark.parametrize("M,N,K,splits,bias", [(1, 256, 320, 1, False), (8, 3584, 18944, 8, False), (37, 896, 4864, 4, True),
                                               (100, 1000, 512, 2, True), (128, 3584, 3584, 8, False), (16, 5120, 13824, 8, False),
                                               (64, 896, 896, 2, False)])
def test_fused_residual_update_and_norm_preparation(M, N, K, splits, bias):
    """The product whose K splits, as one thread-block cluster, add their partial sums into the 32-bit stream through
    each other's shared memory and leave stream * norm weight and the tiles' sums of squares; then the products that finish the norm by scaling their
    output rows.  Against float64: the stream, the RMS, and y = rmsnorm(stream) * weight through each epilogue."""
    from rocmforge_b200.kernels import tensor_core as tc
    eps = 1e-5
    x, w = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=0.05)
    b = rnd(N, seed=3, dt=torch.float32) if bias else None
    nw = (1.0 + 0.3 * rnd(N, seed=4, dt=torch.float32))
    h0 = rnd(M, N, seed=5, dt=torch.float32, scale=2.0)
    want_h = h0.double() + x.double() @ w.double().t() + (b.double() if bias else 0.0)
    outs = []
    for call in range(2):
        h = h0.clone()
        normed, ss = tc.gemm_tc_skinny_resnorm(x, w, b, h, nw, splits=splits)
        close(h, want_h, "stream after the update")
        close(normed, want_h * nw.double(), "stream * norm weight")
        assert tuple(ss.shape) == ((N + 127) // 128, M)
        close(ss.sum(0), (want_h ** 2).sum(1), "sum of squares")
        outs.append((h, normed, ss))
    assert all(torch.equal(a, c) for a, c in zip(outs[0], outs[1])), "the result depends on timing"
    h, normed, ss = outs[1]
    # the finished norm, from the bfloat16 operand that the next product really reads
    y = normed.double() * torch.rsqrt((want_h ** 2).mean(1, keepdim=True) + eps)
    close((y.float()).bfloat16(), want_h * torch.rsqrt((want_h ** 2).mean(1, keepdim=True) + eps) * nw.double(), "finished norm")
    w2, b2 = rnd(384, N, seed=6, scale=0.05), rnd(384, seed=7, dt=torch.float32)
    ref = y @ w2.double().t()
    close(tc.gemm_tc_skinny(normed, w2, mode=tc.F32, row_ss=(ss, eps)), ref, "rows scaled, f32")
    close(tc.gemm_tc_skinny(normed, w2, b2, mode=tc.STORE, row_ss=(ss, eps)), ref + b2.double(), "rows scaled, bias after")
    close(tc.gemm_tc_skinny(normed, w2, mode=tc.SWIGLU, row_ss=(ss, eps)), P.silu(ref[:, 0::2]) * ref[:, 1::2], "rows scaled, swiglu")
    parts = tc.gemm_tc_skinny(normed, w2, mode=tc.PARTIAL, splits=2, row_ss=(ss, eps))
    close(parts.double().sum(0).float(), ref, "rows scaled, partial sums")
    acc = rnd(M, 384, seed=8, dt=torch.float32)
    want = acc.double() + ref
    tc.gemm_tc_skinny(normed, w2, mode=tc.RESIDUAL, out=acc, row_ss=(ss, eps))
    close(acc, want, "rows scaled, residual")
    tc.check_status(DEV)


def test_split_rule_depends_on_the_weight_only():
    from rocmforge_b200.kernels import tensor_core as tc
    assert tc.split_k_for(3584, 3584) > 1 and tc.split_k_for(152064, 3584) == 1
    for N, K in ((3584, 3584), (3584, 18944), (4608, 3584), (896, 4864), (128, 64)):
        s = tc.split_k_for(N, K)
        kb = (K + 63) // 64
        per = (kb + s - 1) // s
        assert s >= 1 and (s - 1) * per < kb


def test_refusals():
    from rocmforge_b200.kernels import tensor_core as tc
    from rocmforge_b200.kernels import KernelError
    assert not tc.supported(4, 8, 12)                  # K * 2 bytes is not a multiple of 16
    with pytest.raises(KernelError):
        tc.gemm_tc(rnd(4, 12), rnd(8, 12))
    with pytest.raises(KernelError):
        tc.gemm_tc_skinny(rnd(tc.SKINNY_MAX_TOKENS + 1, 64), rnd(128, 64))
    with pytest.raises(KernelError):
        tc.gemm_tc(rnd(4, 64, dt=torch.float32), rnd(8, 64, dt=torch.float32))
