"""Models with the layer widths of real checkpoints (few layers, random weights) against the plain model, in
bfloat16 and in the three cuttings (needs a GPU).

The tiny configurations never reach the launch shapes that real widths select: products whose K dimension is
split into partial sums that the rotation kernel or the next norm adds up, seven or five query heads on a kv
head, the clustered product's 224-column tiles with K parts, a vocabulary of 152,064 rows in the output matrix,
a tied output matrix of 151,936 rows.  maeddesg/ROCmForge's closest practice is a whole-model decode against its
CPU path (tests/gpu_decode_real.rs:31-47) at the tolerance of tests/gpu_test_utils.rs:12.

The plain model is the one of tests/plain, reading the same folder; at these widths it keeps the tensors as
stored, widens one at a time to float64 and runs its arithmetic on the GPU (minutes on a CPU otherwise).
"""
import pytest
import torch

from helpers import assert_logits_close, config_dict, random_tokens, write_tiny
from plain.qwen2_plain import PlainModel

pytestmark = pytest.mark.gpu

# layer widths of Qwen2.5-7B, -0.5B and -14B (their config.json values); two layers each
WIDTHS = {
    "7B": dict(seed=11, architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=3584,
               num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
               vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
               max_position_embeddings=1024, use_sliding_window=False),
    "0.5B": dict(seed=12, architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=896,
                 num_attention_heads=14, num_key_value_heads=2, head_dim=64, intermediate_size=4864,
                 vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True,
                 max_position_embeddings=1024, use_sliding_window=False),
    # the 14B vocabulary (152,064 rows of 5,120) is the 7B case again at 1.6 GB more; a smaller one stands here
    "14B": dict(seed=13, architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=5120,
                num_attention_heads=40, num_key_value_heads=8, head_dim=128, intermediate_size=13824,
                vocab_size=8200, rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False,
                max_position_embeddings=1024, use_sliding_window=False),
}
_made = {}


def pair(name, tmp_path_factory):
    """(engine model in bfloat16, plain model) of one folder, made once per session."""
    if name not in _made:
        import rocmforge_b200 as rf
        folder = str(tmp_path_factory.mktemp(f"widths_{name.replace('.', '_')}"))
        write_tiny(WIDTHS[name], folder, "bfloat16", device="cuda:0")      # the same values as on the host, in seconds
        plain = PlainModel(folder, as_stored=True, device="cuda:0")
        _made.clear()                                   # one pair at a time on the device
        torch.cuda.empty_cache()
        _made[name] = (rf.Model.from_folder(folder, dtype=torch.bfloat16), plain)
    return _made[name]


def poison_free_pages(cache):
    for g in cache.groups:
        free = [p for p in range(g.n_pages) if not g.pool.is_held(p)]
        if free:
            g.storage[:, :, torch.tensor(free, device=g.storage.device)] = float("nan")


@pytest.mark.parametrize("name", ["7B", "0.5B", "14B"])
def test_real_widths_in_the_three_cuttings(name, tmp_path_factory):
    from rocmforge_b200 import StepRequest
    from rocmforge_b200.kernels import tensor_core as tc
    m, p = pair(name, tmp_path_factory)
    cfg = WIDTHS[name]
    V, H, I = cfg["vocab_size"], cfg["hidden_size"], cfg["intermediate_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    # the decode schedule of these widths sums partial products: that is what this test is for
    assert tc.split_k_for(qkv, H) > 1 and tc.split_k_for(H, I) > 1

    cache = m.new_cache(max_tokens=64 * 40, max_slots=8)
    # 1. one request whole (logits at a spread of places, the first and the last among them)
    toks = random_tokens(V, 300, 501)
    rows = sorted(set(list(range(0, 300, 37)) + [1, 63, 64, 127, 128, 255, 256, 299]))
    ref = p.logits(toks, rows=rows)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    got = m.step(cache, [StepRequest(s, toks, rows)])
    assert_logits_close(got.cpu(), ref, "bfloat16", f"{name} widths, whole")
    cache.free_slot(s)

    # 2. the same request: a prefix whole, then the last 32 tokens one by one
    poison_free_pages(cache)
    s = cache.alloc_slot()
    assert m.step(cache, [StepRequest(s, toks[:268], [])]) is None
    got = [m.step(cache, [StepRequest(s, [toks[i]], [0])]).cpu() for i in range(268, 300)]
    assert_logits_close(torch.cat(got), p.logits(toks, rows=range(268, 300)), "bfloat16", f"{name} widths, one by one")
    cache.free_slot(s)

    # 3. two batches of eight unequal requests; members end early; the second batch reuses slots and pages
    for b, shapes in enumerate([[(200, 6), (1, 9), (65, 3), (130, 12), (64, 2), (17, 9), (300, 4), (5, 1)],
                                [(128, 5), (3, 8), (257, 2), (40, 8), (90, 6), (64, 7), (2, 3), (33, 8)]]):
        poison_free_pages(cache)
        seqs = [random_tokens(V, plen + dec, 600 + 10 * b + i) for i, (plen, dec) in enumerate(shapes)]
        refs = [p.logits(t, rows=range(plen - 1, plen + dec)) for t, (plen, dec) in zip(seqs, shapes)]
        slots = [cache.alloc_slot() for _ in shapes]
        got = m.step(cache, [StepRequest(sl, t[:plen], [plen - 1]) for sl, t, (plen, _) in zip(slots, seqs, shapes)])
        assert_logits_close(got.cpu(), torch.stack([r[0] for r in refs]), "bfloat16", f"{name} widths, batch {b} prompts")
        live = list(range(len(shapes)))
        step = 0
        while True:
            for i in [i for i in live if shapes[i][1] <= step]:
                cache.free_slot(slots[i])
                live.remove(i)
            if not live:
                break
            poison_free_pages(cache)
            got = m.step(cache, [StepRequest(slots[i], [seqs[i][shapes[i][0] + step]], [0]) for i in live])
            assert_logits_close(got.cpu(), torch.stack([refs[i][1 + step] for i in live]), "bfloat16",
                                f"{name} widths, batch {b} decode step {step}")
            step += 1
        assert cache.live_slots == 0 and all(f == cache.n_pages for f in cache.free_pages())
    tc.check_status(m.device)


def test_ragged_prompts_give_the_same_bits_run_after_run():
    """Sixty-four prompts of 16 to 1,024 tokens in steps of up to 16,384 tokens through all 24 layers of the 0.5B shape,
    run again and again into caches of other sizes and other slots: the logits of every run are those of the first, bit
    for bit, and no kernel's wait ran out.  (With attention grids of several waves and the device busy layer after layer,
    the prompt attention once stood still for its wait's limit, or gave other bits, in one run of ten of this batch;
    two layers, or steps of 2,048 tokens, never showed it.)"""
    import rocmforge_b200 as rf
    from rocmforge_b200 import StepRequest
    from rocmforge_b200.config import Qwen2Config
    from rocmforge_b200.kernels import tensor_core as tc
    _made.clear()
    torch.cuda.empty_cache()
    raw = {k: v for k, v in WIDTHS["0.5B"].items() if k != "seed"}
    raw["num_hidden_layers"] = 24
    m = rf.Model.random(Qwen2Config.from_dict(raw), seed=3, dtype=torch.bfloat16)
    V = raw["vocab_size"]
    g = torch.Generator().manual_seed(4)
    prompts = [random_tokens(V, int(n), 40 + i) for i, n in enumerate(torch.randint(16, 1025, (64,), generator=g).tolist())]
    first = None
    for rep in range(60):
        cache = m.new_cache(max_tokens=sum((len(p) + 64 * (1 + rep % 3)) // 64 * 64 for p in prompts), max_slots=len(prompts))
        slots = [cache.alloc_slot() for _ in prompts]
        if rep % 2:
            slots = slots[::-1]
        outs, i = [], 0
        while i < len(prompts):
            j, t = i, 0
            while j < len(prompts) and (j == i or t + len(prompts[j]) <= 16384):
                t += len(prompts[j])
                j += 1
            outs.append(m.step(cache, [StepRequest(s, p, [len(p) - 1]) for s, p in zip(slots[i:j], prompts[i:j])]))
            i = j
        got = torch.cat(outs)
        tc.check_status(m.device)
        if first is None:
            first = got.clone()
        assert torch.equal(got, first), f"run {rep} gave other logits than the first"
        del cache


@pytest.mark.parametrize("name", ["7B", "0.5B"])
def test_real_widths_with_norms_prepared_by_the_product_before_them(name, tmp_path_factory):
    """``Options.fused_norm``: the o and down products of few tokens add their K splits into the stream themselves and
    leave the next norm half done; q|k|v and gate/up finish it by scaling their output rows.  Decoding and a short
    appended chunk at real widths (10 and 19 splits) against the plain model."""
    from rocmforge_b200 import StepRequest
    m, p = pair(name, tmp_path_factory)
    V = WIDTHS[name]["vocab_size"]
    m.options.fused_norm = True
    try:
        cache = m.new_cache(max_tokens=64 * 16, max_slots=4)
        poison_free_pages(cache)
        seqs = [random_tokens(V, n, 800 + n) for n in (150, 90, 33)]
        refs = [p.logits(t, rows=range(len(t) - 25, len(t))) for t in seqs]
        slots = [cache.alloc_slot() for _ in seqs]
        m.step(cache, [StepRequest(s, t[:-25], []) for s, t in zip(slots, seqs)])
        got = m.step(cache, [StepRequest(s, t[-25:-20], range(5)) for s, t in zip(slots, seqs)])       # 15 tokens a step
        assert_logits_close(got.cpu(), torch.cat([r[:5] for r in refs]), "bfloat16", f"{name} fused norm, chunks")
        for k in range(20):
            got = m.step(cache, [StepRequest(s, [t[len(t) - 20 + k]], [0]) for s, t in zip(slots, seqs)])
            assert_logits_close(got.cpu(), torch.stack([r[5 + k] for r in refs]), "bfloat16", f"{name} fused norm, step {k}")
    finally:
        m.options.fused_norm = False


@pytest.mark.parametrize("name", ["7B", "0.5B"])
def test_real_widths_device_loop_follows_the_plain_loop(name, tmp_path_factory):
    """The replayed greedy loop (graph per step, ids fed back on the device) at real widths: its tokens are the
    plain loop's up to the first near tie of bfloat16."""
    from rocmforge_b200 import StepRequest, kernels
    from rocmforge_b200.engine.graph import DecodeRunner
    from plain import sampling_plain as S
    from test_engine_gpu import check_tokens_up_to_near_ties
    m, p = pair(name, tmp_path_factory)
    V = WIDTHS[name]["vocab_size"]
    prompts = [random_tokens(V, n, 700 + n) for n in (61, 20, 3)]
    cache = m.new_cache(max_tokens=64 * 8, max_slots=4)
    poison_free_pages(cache)
    runner = DecodeRunner(m, cache)
    slots = [cache.alloc_slot() for _ in prompts]
    first = kernels.argmax(m.step(cache, [StepRequest(s, t, [len(t) - 1]) for s, t in zip(slots, prompts)])).cpu().tolist()
    ids, _, _, _ = runner.greedy_loop(slots, first, 10)
    got = torch.cat([torch.tensor([first], dtype=torch.int32), ids.cpu()]).t().tolist()
    for i, pr in enumerate(prompts):
        want, _ = S.generate(lambda t: p.logits(t, rows=[len(t) - 1])[0], pr, max_tokens=11)
        check_tokens_up_to_near_ties(p, pr, got[i], want)
