"""Launch shapes that are chosen on the host: they depend on sizes alone, never on timing or on the data."""
from rocmforge_b200.kernels import basic
from rocmforge_b200.kernels import tensor_core as tc


def test_k_splits_depend_on_the_weight_shape_and_the_token_bucket():
    # Qwen2.5-7B layer shapes: about two CTAs per SM, every split at least four blocks of 64
    assert tc.split_k_for(37888, 3584) == 1            # 296 tiles fill the GPU without a split
    for N, K in ((4608, 3584), (3584, 3584), (3584, 18944), (152064, 3584), (128, 64), (1000, 200)):
        s = tc.split_k_for(N, K)
        kb = (K + 63) // 64
        per = (kb + s - 1) // s
        assert s >= 1 and (s - 1) * per < kb, "no split is empty"
        assert s == 1 or kb // s >= 4
        tiles = (N + 127) // 128
        assert s == 1 or tiles * s <= 2 * 148, "a split product stays within two CTAs per SM"
        # a step of at most 16 tokens fits three CTAs on an SM: long K ranges are then cut finer, short ones stay
        few = tc.split_k_for(N, K, tokens=8)
        assert few >= s and (few == s or (tiles * few <= 3 * 148 and kb // few >= 16))
        assert tc.split_k_for(N, K, tokens=17) == s and tc.split_k_for(N, K, tokens=128) == s
    assert tc.split_k_for(3584, 18944, tokens=1) == 15 and tc.split_k_for(3584, 18944) == 10
    assert tc.split_k_for(4608, 3584, tokens=1) == 8 and tc.split_k_for(3584, 3584, tokens=16) == 10


def test_decode_cluster_size_from_batch_and_context():
    # one CTA per SM or so, never more CTAs than pages, 16 only for a single sequence with a long context
    assert basic.decode_splits(1, 4) == 8
    assert basic.decode_splits(8, 4) == 4
    assert basic.decode_splits(16, 4) == 2
    assert basic.decode_splits(64, 4) == 1
    assert basic.decode_splits(1, 4, longest=64) == 1
    assert basic.decode_splits(1, 4, longest=100) == 2
    assert basic.decode_splits(1, 4, longest=4096) == 16
    assert basic.decode_splits(1, 8, longest=4096) == 8
    assert basic.decode_splits(2, 4, longest=4096) == 8
    assert basic.decode_splits(1, 4, longest=1 << 20, window=128) == 2
    for B in (1, 2, 3, 5, 8, 13, 64, 300):
        for nkv in (1, 2, 4, 8, 40):
            for longest in (1, 63, 64, 65, 1000, 100000):
                s = basic.decode_splits(B, nkv, longest)
                assert s in (1, 2, 4, 8, 16) and s <= max(1, basic.decode_pages(longest, None))


def test_pages_a_new_token_reads():
    assert basic.decode_pages(1, None) == 1 and basic.decode_pages(64, None) == 1 and basic.decode_pages(65, None) == 2
    assert basic.decode_pages(1 << 20, 1024) == 17      # a window of 1,024 keys touches at most 17 pages of 64
    assert basic.decode_pages(100, 1024) == 2


def test_decode_descriptor_fits_the_runner_at_its_largest_batch():
    """A runner's device descriptor is sized once and never moved (captured graphs keep its address): the packed
    descriptor of the largest decode batch, tile tables included, must fit it."""
    from rocmforge_b200.engine.batch import StepBatch, StepRequest
    from rocmforge_b200.engine.graph import DecodeRunner
    for max_batch in (1, 64, 683, 1024):
        reqs = [StepRequest(i, [1], [0]) for i in range(max_batch)]
        packed = StepBatch(reqs, [5] * max_batch, vocab_size=10).pack()
        assert packed.size <= DecodeRunner.descriptor_words(max_batch)
