"""The engine against the plain implementation, in 32-bit and in bfloat16 (needs a GPU)."""
import math
import os

import numpy as np
import pytest
import torch

from helpers import CONFIGS, TraceRun, assert_logits_close, random_tokens
from plain.qwen2_plain import PlainModel
from plain import sampling_plain as S

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_models, _plains = {}, {}


def engine(folders, name, dtype, **opts):
    import rocmforge_b200 as rf
    key = (name, dtype, tuple(sorted(opts.items())))
    if key not in _models:
        _models[key] = rf.Model.from_folder(folders(name, dtype), dtype=TORCH[dtype],
                                            options=rf.Options(**opts) if opts else None)
    return _models[key]


def plain(folders, name, dtype):
    key = (name, dtype)
    if key not in _plains:
        _plains[key] = PlainModel(folders(name, dtype))       # the same stored (rounded) weights
    return _plains[key]


def poison_free_pages(cache):
    """Fill every page no sequence holds with NaN: a kernel that reads a stale page shows it."""
    for g in cache.groups:
        free = [p for p in range(g.n_pages) if not g.pool.is_held(p)]
        if free:
            g.storage[:, :, torch.tensor(free, device=g.storage.device)] = float("nan")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["D", "E"])
def test_a_prompt_of_more_than_512_tokens(folders, name, dtype):
    """From 512 rows on a prompt step's norm takes a kernel of its own, its attention walks ten and more pages per
    query tile (E: a window of 200 far behind the newest token), and two prompts in one step share the tile table.
    Logits at a spread of places, then a few decoded tokens, against the plain model."""
    from rocmforge_b200 import StepRequest
    m, p = engine(folders, name, dtype), plain(folders, name, dtype)
    V = CONFIGS[name]["vocab_size"]
    cache = m.new_cache(max_tokens=64 * 26, max_slots=4)
    poison_free_pages(cache)
    a, b = random_tokens(V, 700, 41), random_tokens(V, 530, 42)
    ra, rb = p.logits(a), p.logits(b)
    sa, sb = cache.alloc_slot(), cache.alloc_slot()
    wa, wb = [0, 1, 63, 64, 199, 200, 201, 511, 512, 513, 639, 640, 689], [0, 255, 256, 511, 512, 519]
    got = m.step(cache, [StepRequest(sa, a[:690], wa), StepRequest(sb, b[:520], wb)]).cpu()
    assert_logits_close(got, torch.cat([ra[wa], rb[wb]]), dtype, f"{name} {dtype} two long prompts")
    for k in range(10):
        got = m.step(cache, [StepRequest(sa, [a[690 + k]], [0]), StepRequest(sb, [b[520 + k]], [0])]).cpu()
        assert_logits_close(got, torch.stack([ra[690 + k], rb[520 + k]]), dtype, f"{name} {dtype} decode {k} after long prompts")
    cache.free_slot(sa); cache.free_slot(sb)
    assert cache.live_slots == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["D", "E"])
def test_tuned_kernel_paths_prompt_chunk_decode_and_batch(folders, name, dtype):
    """Sizes at which the bfloat16 engine runs its tensor-core products (clustered for >= 256 rows), the tiled
    prefill attention and the chunked decode attention: a 300-token prompt, a chunk, decoding across page and
    chunk borders, then a ragged batch that reuses the pages."""
    from rocmforge_b200 import StepRequest
    m, p = engine(folders, name, dtype), plain(folders, name, dtype)
    V = CONFIGS[name]["vocab_size"]
    cache = m.new_cache(max_tokens=64 * 16, max_slots=4)
    toks = random_tokens(V, 420, 31)
    ref = p.logits(toks)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    got = [m.step(cache, [StepRequest(s, toks[:300], range(300))]).cpu(),
           m.step(cache, [StepRequest(s, toks[300:380], range(80))]).cpu()]
    for i in range(380, 420):
        got.append(m.step(cache, [StepRequest(s, [toks[i]], [0])]).cpu())
    assert_logits_close(torch.cat(got), ref, dtype, f"{name} {dtype} prompt + chunk + decode")
    cache.free_slot(s)
    poison_free_pages(cache)
    lens = [(257, 20), (70, 30), (1, 40), (130, 5)]
    seqs = [random_tokens(V, a + b, 50 + i) for i, (a, b) in enumerate(lens)]
    refs = [p.logits(t) for t in seqs]
    slots = [cache.alloc_slot() for _ in lens]
    got = m.step(cache, [StepRequest(sl, t[:a], [a - 1]) for sl, t, (a, _) in zip(slots, seqs, lens)])
    assert_logits_close(got.cpu(), torch.stack([r[a - 1] for r, (a, _) in zip(refs, lens)]), dtype, f"{name} ragged prompts")
    live = list(range(4))
    for step in range(40):
        for i in [i for i in live if lens[i][1] <= step]:
            cache.free_slot(slots[i]); live.remove(i)
        got = m.step(cache, [StepRequest(slots[i], [seqs[i][lens[i][0] + step]], [0]) for i in live])
        assert_logits_close(got.cpu(), torch.stack([refs[i][lens[i][0] + step] for i in live]), dtype,
                            f"{name} batch decode step {step}")


@pytest.mark.parametrize("option", ["clustered_decode", "tcgen05_attention", "tuned_attention", "tensor_core_gemm",
                                    "fused_norm"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_every_switch_of_the_engine_keeps_the_results(folders, name, option):
    """Each option flipped takes another kernel for the same step (the chunked decode attention, the mma.sync
    prefill attention, the generic attention, the CUDA-core products; norms prepared by the product before them):
    same logits as the plain model."""
    import rocmforge_b200 as rf
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, "bfloat16", **{option: not getattr(rf.Options(), option)})
    p = plain(folders, name, "bfloat16")
    V = CONFIGS[name]["vocab_size"]
    cache = m.new_cache(max_tokens=64 * 12, max_slots=2)
    seqs = [random_tokens(V, 330, 71), random_tokens(V, 150, 72)]
    refs = [p.logits(t) for t in seqs]
    poison_free_pages(cache)
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    cut = [300, 120]
    got = m.step(cache, [StepRequest(sl, t[:c], range(c)) for sl, t, c in zip(slots, seqs, cut)])
    assert_logits_close(got.cpu(), torch.cat([r[:c] for r, c in zip(refs, cut)]), "bfloat16", f"{name} {option}=False prompts")
    for step in range(30):
        got = m.step(cache, [StepRequest(sl, [t[c + step]], [0]) for sl, t, c in zip(slots, seqs, cut)])
        assert_logits_close(got.cpu(), torch.stack([r[c + step] for r, c in zip(refs, cut)]), "bfloat16",
                            f"{name} {option}=False decode step {step}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_each_request_alone_and_whole(folders, name, dtype):
    from rocmforge_b200 import StepRequest
    m, p = engine(folders, name, dtype), plain(folders, name, dtype)
    cache = m.new_cache(max_tokens=256)
    for n, seed in ((1, 1), (2, 2), (63, 3), (64, 4), (65, 5), (100, 6)):
        toks = random_tokens(CONFIGS[name]["vocab_size"], n, seed)
        poison_free_pages(cache)
        s = cache.alloc_slot()
        got = m.step(cache, [StepRequest(s, toks, range(n))])
        assert_logits_close(got.cpu(), p.logits(toks), dtype, f"{name} {dtype} whole n={n}")
        cache.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_last_32_tokens_one_by_one(folders, name, dtype):
    from rocmforge_b200 import StepRequest
    m, p = engine(folders, name, dtype), plain(folders, name, dtype)
    cache = m.new_cache(max_tokens=256)
    toks = random_tokens(CONFIGS[name]["vocab_size"], 90, 21)
    ref = p.logits(toks)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    got = [m.step(cache, [StepRequest(s, toks[:58], range(58))]).cpu()]
    for i in range(58, 90):
        got.append(m.step(cache, [StepRequest(s, [toks[i]], [0])]).cpu())
        assert cache.length(s) == i + 1
    assert_logits_close(torch.cat(got), ref, dtype, f"{name} {dtype} last 32 one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_one_after_another(folders, name, dtype):
    """Prompts of unequal lengths in one step, then one token each; shorter requests end earlier;
    the next batch reuses the slots and pages, which are poisoned in between."""
    from rocmforge_b200 import StepRequest
    m, p = engine(folders, name, dtype), plain(folders, name, dtype)
    V = CONFIGS[name]["vocab_size"]
    cache = m.new_cache(max_tokens=64 * 7, max_slots=4)
    used_slots = []
    for b, shapes in enumerate([[(5, 9), (40, 3), (1, 12), (70, 30)], [(64, 2), (3, 40), (17, 17)],
                                [(90, 10), (2, 2), (33, 31), (1, 1)]]):
        poison_free_pages(cache)
        seqs = [random_tokens(V, plen + dec, 100 * b + i) for i, (plen, dec) in enumerate(shapes)]
        refs = [p.logits(t) for t in seqs]
        slots = [cache.alloc_slot() for _ in shapes]
        used_slots.append(tuple(slots))
        got = m.step(cache, [StepRequest(s, t[:plen], range(plen)) for s, t, (plen, _) in zip(slots, seqs, shapes)])
        off = 0
        for i, (plen, _) in enumerate(shapes):
            assert_logits_close(got[off:off + plen].cpu(), refs[i][:plen], dtype, f"{name} batch {b} prompt {i}")
            off += plen
        live = list(range(len(shapes)))
        step = 0
        while live:
            # requests whose tokens are used up end here and give their slot back
            for i in [i for i in live if shapes[i][1] <= step]:
                cache.free_slot(slots[i])
                live.remove(i)
            if not live:
                break
            poison_free_pages(cache)
            got = m.step(cache, [StepRequest(slots[i], [seqs[i][shapes[i][0] + step]], [0]) for i in live])
            for row, i in enumerate(live):
                at = shapes[i][0] + step
                assert_logits_close(got[row:row + 1].cpu(), refs[i][at:at + 1], dtype,
                                    f"{name} batch {b} request {i} decode step {step}")
            step += 1
        assert cache.live_slots == 0 and all(f == cache.n_pages for f in cache.free_pages())
    assert used_slots[0] == used_slots[2], "the slots of a finished batch are used again"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "C"])
def test_long_decoding(folders, name, dtype):
    from rocmforge_b200 import StepRequest
    m, p = engine(folders, name, dtype), plain(folders, name, dtype)
    n = 250
    toks = random_tokens(CONFIGS[name]["vocab_size"], n, 77)
    ref = p.logits(toks)
    cache = m.new_cache(max_tokens=256)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    got = [m.step(cache, [StepRequest(s, toks[:3], range(3))]).cpu()]
    for i in range(3, n):
        got.append(m.step(cache, [StepRequest(s, [toks[i]], [0])]).cpu())
    assert_logits_close(torch.cat(got), ref, dtype, f"{name} {dtype} long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(folders, dtype):
    from rocmforge_b200 import StepRequest
    m, p = engine(folders, "A", dtype), plain(folders, "A", dtype)
    cache = m.new_cache(max_tokens=256)
    toks = random_tokens(256, 4, 5)
    ref = p.logits(toks)
    s = cache.alloc_slot()
    for i, t in enumerate(toks):           # from the very first token on, one at a time
        got = m.step(cache, [StepRequest(s, [t], [0])])
        assert_logits_close(got.cpu(), ref[i:i + 1], dtype, f"first tokens, position {i}")
    # logits only where wanted, in the order asked for
    s2 = cache.alloc_slot()
    got = m.step(cache, [StepRequest(s2, toks, [3, 0])])
    assert_logits_close(got.cpu(), ref[[3, 0]], dtype, "wanted rows in the order given")
    s3 = cache.alloc_slot()
    assert m.step(cache, [StepRequest(s3, toks, [])]) is None and cache.length(s3) == 4


@pytest.mark.parametrize("dtype", DTYPES)
def test_chunked_prompt(folders, dtype):
    """Several tokens appended to an existing context in one step."""
    from rocmforge_b200 import StepRequest
    m, p = engine(folders, "C", dtype), plain(folders, "C", dtype)
    toks = random_tokens(300, 150, 9)
    ref = p.logits(toks)
    cache = m.new_cache(max_tokens=256)
    s = cache.alloc_slot()
    got, at = [], 0
    for n in (10, 54, 1, 63, 22):
        got.append(m.step(cache, [StepRequest(s, toks[at:at + n], range(n))]).cpu())
        at += n
    assert_logits_close(torch.cat(got), ref, dtype, "prompt in chunks")


def test_step_refuses_bad_input(folders):
    from rocmforge_b200 import StepRequest, CacheError
    from rocmforge_b200.engine import BatchError
    m = engine(folders, "A", "float32")
    cache = m.new_cache(max_tokens=128)
    s = cache.alloc_slot()
    with pytest.raises(BatchError):
        m.step(cache, [StepRequest(s, [1, 256], [0])])          # id outside the vocabulary
    with pytest.raises(BatchError):
        m.step(cache, [StepRequest(s, [], [])])
    with pytest.raises(BatchError):
        m.step(cache, [StepRequest(s, [1], [1])])               # wanted place beyond the tokens
    with pytest.raises(CacheError):
        m.step(cache, [StepRequest(s, [1], [0]), StepRequest(s, [2], [0])])
    with pytest.raises(CacheError):
        m.step(cache, [StepRequest(3, [1], [0])])               # slot nobody holds
    with pytest.raises(CacheError):
        m.step(cache, [StepRequest(s, list(range(129)), [])])   # beyond max_position_embeddings
    assert cache.length(s) == 0 and cache.free_pages() == [cache.n_pages]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_trace_run_three_cuttings(folders, name, dtype, tmp_path):
    """bin/trace_run as a child process: whole, last 32 one by one, unequal batches with reuse."""
    p = plain(folders, name, dtype)
    V = CONFIGS[name]["vocab_size"]
    seqs = {rid: random_tokens(V, n, 300 + i) for i, (rid, n) in
            enumerate([("w1", 70), ("w2", 33), ("d", 100), ("b1", 12), ("b2", 80), ("b3", 45), ("c1", 64), ("c2", 7)])}
    refs = {rid: p.logits(t) for rid, t in seqs.items()}
    tr = TraceRun(folders(name, dtype), dtype, str(tmp_path / "out"), max_tokens=64 * 5)
    # 1. whole
    for rid in ("w1", "w2"):
        got = tr.step([(rid, seqs[rid], range(len(seqs[rid])))], end=[rid])
        assert_logits_close(got, refs[rid], dtype, f"trace whole {rid}")
    # 2. prefix, then the last 32 one by one; nothing wanted in the prefix step
    assert tr.step([("d", seqs["d"][:68], [])]) is None
    for i in range(68, 100):
        got = tr.step([("d", [seqs["d"][i]], [0])], end=["d"] if i == 99 else [])
        assert_logits_close(got, refs["d"][i:i + 1], dtype, f"trace decode at {i}")
    # 3. two batches of unequal lengths; shorter requests end earlier; slots and pages are reused
    for ids, plens in ((("b1", "b2", "b3"), (4, 60, 30)), (("c1", "c2"), (50, 3))):
        got = tr.step([(r, seqs[r][:n], [n - 1]) for r, n in zip(ids, plens)])
        assert_logits_close(got, torch.stack([refs[r][n - 1] for r, n in zip(ids, plens)]), dtype, "trace batch prompts")
        at = dict(zip(ids, plens))
        live = list(ids)
        while live:
            ending = [r for r in live if at[r] + 1 == len(seqs[r])]
            got = tr.step([(r, [seqs[r][at[r]]], [0]) for r in live], end=ending)
            assert_logits_close(got, torch.stack([refs[r][at[r]] for r in live]), dtype, "trace batch decode")
            for r in live:
                at[r] += 1
            live = [r for r in live if r not in ending]
    assert tr.close() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(folders, dtype):
    import rocmforge_b200 as rf
    p = plain(folders, "A", dtype)
    llm = rf.LLM(folders("A", dtype), dtype=dtype, max_batch=2)
    prompts = [random_tokens(256, n, 40 + n) for n in (5, 9, 12)]            # 3 requests, batches of 2
    out = llm.generate(prompts, max_tokens=8, temperature=0.0, stop_token_ids=[])
    for i, (pr, r) in enumerate(zip(prompts, out)):
        want, reason = S.generate(lambda t: p.logits(t)[-1], pr, max_tokens=8)
        if dtype == "float32":
            assert r.tokens == want and r.reason == reason, f"request {i}"
        else:
            check_tokens_up_to_near_ties(p, pr, r.tokens, want)
    assert llm.cache.live_slots == 0
    # stop tokens and the context limit (max_position_embeddings = 128)
    first = out[0].tokens
    again = llm.generate(prompts[:1], max_tokens=8, temperature=0.0, stop_token_ids=[first[3]])
    assert again[0].tokens == first[:first.index(first[3])] and again[0].reason == "stop_token"
    long = llm.generate([random_tokens(256, 125, 1)], max_tokens=50, temperature=0.0, stop_token_ids=[])
    assert len(long[0].tokens) == 3 and long[0].reason == "context_full"


def check_tokens_up_to_near_ties(p, prompt, got, want):
    """bfloat16 may flip an argmax whose two best logits are closer than its error bound;
    up to the first such place the tokens must agree."""
    toks = list(prompt)
    for g, w in zip(got, want):
        if g != w:
            last = p.logits(toks)[-1]
            top2 = torch.topk(last, 2).values
            assert float(top2[0] - top2[1]) < 2e-2 * float(last.abs().max()), "tokens differ without a near tie"
            return
        toks.append(g)


def check_sampled_up_to_swapped_neighbours(p, prompt, got, want, temperature):
    """Sampled tokens must be the plain sampler's.  The sampler walks the tokens in the order of their probabilities;
    two tokens whose probabilities agree to seven digits may stand in either order, and a draw that lands on them then
    picks the one or the other: up to the first such place the tokens must agree, and there the two candidates must
    be such a pair."""
    toks = list(prompt)
    for k, (g, w) in enumerate(zip(got, want)):
        if g != w:
            pr = torch.softmax(p.logits(toks)[-1].double() / temperature, dim=0)
            assert abs(float(pr[g] - pr[w])) < 1e-6 * float(pr[w]), f"token {k}: {g} instead of {w} without a tie in the order"
            return
        toks.append(g)
    assert len(got) == len(want)


def test_sampled_generation_follows_the_plain_sampler(folders):
    """Tiny B, temperature 0.8, seeded: a batch of 4 with prompt lengths 1/7/16/31, 6 steps."""
    import rocmforge_b200 as rf
    p = plain(folders, "B", "float32")
    llm = rf.LLM(folders("B", "float32"), dtype="float32")
    prompts = [random_tokens(384, n, 60 + n) for n in (1, 7, 16, 31)]
    for kw in (dict(temperature=0.8, top_p=1.0), dict(temperature=0.8, top_p=0.9),
               dict(temperature=1.3, top_p=0.95, top_k=20)):
        out = llm.generate(prompts, max_tokens=6, seed=1, stop_token_ids=[], **kw)
        for i, (pr, r) in enumerate(zip(prompts, out)):
            want, _ = S.generate(lambda t: p.logits(t)[-1].float(), pr, max_tokens=6, seed=1, request=i,
                                 top_k=kw.get("top_k", 0), temperature=kw["temperature"], top_p=kw["top_p"])
            check_sampled_up_to_swapped_neighbours(p, pr, r.tokens, want, kw["temperature"])
    # a request's draws do not depend on its neighbours
    alone = llm.generate(prompts[:1], max_tokens=6, seed=1, temperature=0.8, top_p=1.0, stop_token_ids=[])
    both = llm.generate(prompts[:2], max_tokens=6, seed=1, temperature=0.8, top_p=1.0, stop_token_ids=[])
    assert alone[0].tokens == both[0].tokens


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["C", "D"])
def test_graph_replay_equals_plain_steps(folders, name, dtype):
    import rocmforge_b200 as rf
    prompts = [random_tokens(300, n, n) for n in (3, 30, 64)]
    a = rf.LLM(folders(name, dtype), dtype=dtype, options=rf.Options(decode_graphs=True))
    b = rf.LLM(folders(name, dtype), dtype=dtype, options=rf.Options(decode_graphs=False))
    ra = a.generate(prompts, max_tokens=70, temperature=0.0, stop_token_ids=[])
    rb = b.generate(prompts, max_tokens=70, temperature=0.0, stop_token_ids=[])
    assert a.engine.decode_runner.replays > 0 and b.engine.decode_runner is None
    assert [r.tokens for r in ra] == [r.tokens for r in rb]


def test_graph_decode_across_length_buckets(folders):
    """Replayed decode steps whose graphs are captured per (batch, length bucket): sequences that grow from under 512 keys to
    over it (a window of 200 in one layer), the shorter ones ending earlier, against the plain model."""
    from rocmforge_b200 import StepRequest
    from rocmforge_b200.engine.graph import DecodeRunner
    m, p = engine(folders, "E", "bfloat16"), plain(folders, "E", "bfloat16")
    V = CONFIGS["E"]["vocab_size"]
    lens = [(450, 120), (500, 40), (440, 30)]
    seqs = [random_tokens(V, a + b, 300 + i) for i, (a, b) in enumerate(lens)]
    refs = [p.logits(t) for t in seqs]
    cache = m.new_cache(max_tokens=64 * 40, max_slots=4)
    poison_free_pages(cache)
    runner = DecodeRunner(m, cache)
    slots = [cache.alloc_slot() for _ in lens]
    m.step(cache, [StepRequest(s, t[:a], []) for s, t, (a, _) in zip(slots, seqs, lens)])
    live = list(range(len(lens)))
    for step in range(max(b for _, b in lens)):
        for i in [i for i in live if lens[i][1] <= step]:
            cache.free_slot(slots[i]); live.remove(i)
        got = runner.logits([slots[i] for i in live], [seqs[i][lens[i][0] + step] for i in live]).cpu()
        assert_logits_close(got, torch.stack([refs[i][lens[i][0] + step] for i in live]), "bfloat16", f"step {step}")
    assert {k[1] for k in runner.graphs} >= {512, 1024}
