"""The replayed decode paths of ``DecodeRunner`` against the plain model (needs a GPU): the loop that feeds the
sampled ids back on the device, and the step that is prepared ahead of time while slots come and go."""
import pytest
import torch

from helpers import CONFIGS, assert_logits_close, random_tokens
from plain import sampling_plain as S
from test_engine_gpu import (check_sampled_up_to_swapped_neighbours, check_tokens_up_to_near_ties, engine, plain,
                             poison_free_pages)

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype,plens,steps", [
    ("A", "float32", (5, 60, 63), 40),           # across the border of a 64-position page
    ("A", "bfloat16", (5, 60, 63), 40),
    ("D", "float32", (470, 481, 3), 60),         # across a page border and the 512-key bound of a captured graph
    ("D", "bfloat16", (470, 481, 3), 60)])
def test_greedy_loop_on_the_device_gives_the_tokens_of_generate_and_of_the_plain_loop(folders, name, dtype, plens, steps):
    """``greedy_loop`` replays one graph per step (forward, argmax, advance of tokens and positions, all on the
    device).  Its ids must be those of ``LLM.generate(temperature=0)`` and of the plain loop; a position that did
    not advance, or a page that was not reserved, changes them."""
    import rocmforge_b200 as rf
    from rocmforge_b200 import StepRequest, kernels
    from rocmforge_b200.engine.graph import DecodeRunner
    m, p = engine(folders, name, dtype), plain(folders, name, dtype)
    V = CONFIGS[name]["vocab_size"]
    prompts = [random_tokens(V, n, 900 + n) for n in plens]
    cache = m.new_cache(max_tokens=64 * 30, max_slots=4)
    poison_free_pages(cache)
    runner = DecodeRunner(m, cache)
    slots = [cache.alloc_slot() for _ in prompts]
    logits = m.step(cache, [StepRequest(s, t, [len(t) - 1]) for s, t in zip(slots, prompts)])
    first = kernels.argmax(logits).cpu().tolist()
    # two loops one after the other: the second starts where the first stopped (descriptor uploaded anew)
    ids_a, _, _, _ = runner.greedy_loop(slots, first, steps // 2)
    ids_b, _, _, launches = runner.greedy_loop(slots, ids_a[-1].cpu().tolist(), steps - steps // 2)
    got = torch.cat([torch.tensor([first], dtype=torch.int32), ids_a.cpu(), ids_b.cpu()]).t().tolist()   # [request][1 + steps]
    assert launches > 0 and all(cache.length(s) == n + steps for s, n in zip(slots, plens))
    if name == "D":
        assert {k[2] for k in runner.graphs if k[0] == "loop"} >= {512, 1024}
    llm = rf.LLM(m, max_batch=4)
    out = llm.generate(prompts, max_tokens=steps + 1, temperature=0.0, stop_token_ids=[])
    for i, (pr, r) in enumerate(zip(prompts, out)):
        want, _ = S.generate(lambda t: p.logits(t)[-1], pr, max_tokens=steps + 1)
        if dtype == "float32":
            assert got[i] == want, f"request {i}: the device loop left the plain loop"
            assert r.tokens == want, f"request {i}: generate() left the plain loop"
        else:
            check_tokens_up_to_near_ties(p, pr, got[i], want)
            check_tokens_up_to_near_ties(p, pr, r.tokens, want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_prepared_ahead_is_dropped_when_slots_change(folders, dtype):
    """The runner prepares the next step of a batch (pages, positions) while the device works.  Two sequences end
    at 64 and 128 tokens, exactly on page borders, after the runner took the pages for their next positions; their
    slots are freed and filled again with prompts of 64 and 128 tokens while a third sequence lives on (so the
    free list hands out other pages).  Slots and lengths are as the prepared step has them, the pages are not:
    the runner must build the step anew.  Free pages are poisoned; logits against the plain model."""
    from rocmforge_b200 import StepRequest
    from rocmforge_b200.engine.graph import DecodeRunner
    m, p = engine(folders, "D", dtype), plain(folders, "D", dtype)
    V = CONFIGS["D"]["vocab_size"]
    cache = m.new_cache(max_tokens=64 * 16, max_slots=4)
    runner = DecodeRunner(m, cache)
    keep_toks = random_tokens(V, 120, 1)
    keep = cache.alloc_slot()
    m.step(cache, [StepRequest(keep, keep_toks[:70], [])])
    # batch 1: ends at lengths 64 and 128 through the runner
    first = [random_tokens(V, 64, 2), random_tokens(V, 128, 3)]
    refs1 = [p.logits(t) for t in first]
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    m.step(cache, [StepRequest(s, t[:-4], []) for s, t in zip(slots, first)])
    for k in range(4):
        got = runner.logits(slots, [t[len(t) - 4 + k] for t in first]).cpu()
        assert_logits_close(got, torch.stack([r[len(r) - 4 + k] for r in refs1]), dtype, f"batch 1 step {k}")
    assert [cache.length(s) for s in slots] == [64, 128]
    assert runner._ready is not None, "the runner has the next step of this batch prepared"
    for s in slots:
        cache.free_slot(s)
    # the third sequence grows meanwhile and takes the lowest free pages
    m.step(cache, [StepRequest(keep, keep_toks[70:100], [])])
    # batch 2: the same slots, prompts of the same lengths
    second = [random_tokens(V, 64 + 12, 4), random_tokens(V, 128 + 12, 5)]
    refs2 = [p.logits(t) for t in second]
    again = [cache.alloc_slot(), cache.alloc_slot()]
    assert again == slots
    m.step(cache, [StepRequest(s, t[:n], []) for s, t, n in zip(again, second, (64, 128))])
    poison_free_pages(cache)
    for k in range(10):
        poison_free_pages(cache)
        got = runner.logits(again, [t[n + k] for t, n in zip(second, (64, 128))]).cpu()
        assert_logits_close(got, torch.stack([r[n + k] for r, n in zip(refs2, (64, 128))]), dtype, f"batch 2 step {k}")
    # and the sequence that lived through both batches is intact
    ref = p.logits(keep_toks)
    for i in range(100, 120):
        got = m.step(cache, [StepRequest(keep, [keep_toks[i]], [0])]).cpu()
        assert_logits_close(got, ref[i:i + 1], dtype, f"the third sequence at {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_of_the_host_follow_the_plain_loop(folders, dtype):
    """``step_ids`` keeps the device one step ahead: the next step's tokens are gathered on the device from the ids
    the host has not seen yet.  Sequences stop at different times (their rows of the step that ran ahead are
    ignored, the others go on without a relaunch), one call passes other tokens than it was given (the step that ran
    ahead is dropped and its page given back), and a slot is freed and refilled between two calls."""
    from rocmforge_b200 import SamplingParams, StepRequest, kernels
    from rocmforge_b200.engine.graph import DecodeRunner
    m, p = engine(folders, "D", dtype), plain(folders, "D", dtype)
    V = CONFIGS["D"]["vocab_size"]
    greedy = SamplingParams(temperature=0.0)
    cache = m.new_cache(max_tokens=64 * 24, max_slots=4)
    poison_free_pages(cache)
    runner = DecodeRunner(m, cache)
    prompts = [random_tokens(V, n, 950 + n) for n in (62, 127, 5)]
    budget = [9, 30, 20]                                   # tokens each request may take: they stop at different times
    want = [S.generate(lambda t: p.logits(t)[-1], pr, max_tokens=b)[0] for pr, b in zip(prompts, budget)]
    slots = [cache.alloc_slot() for _ in prompts]
    first = kernels.argmax(m.step(cache, [StepRequest(s, t, [len(t) - 1]) for s, t in zip(slots, prompts)])).cpu().tolist()
    got = [[f] for f in first]
    live = [0, 1, 2]
    while True:
        for i in [i for i in live if len(got[i]) >= budget[i]]:
            cache.free_slot(slots[i])
            live.remove(i)
        if not live:
            break
        poison_free_pages(cache)
        ids = runner.step_ids([slots[i] for i in live], [got[i][-1] for i in live], greedy, live,
                              [len(got[i]) for i in live])             # request numbers and the count of each one's draws
        for i, t in zip(live, ids):
            got[i].append(t)
    assert runner.launched_ahead >= 20, "the steps did not run ahead of the host"
    for i in range(3):
        if dtype == "float32":
            assert got[i] == want[i], f"request {i}"
        else:
            check_tokens_up_to_near_ties(p, prompts[i], got[i], want[i])
    assert cache.live_slots == 0 and all(f == cache.n_pages for f in cache.free_pages()), "a page taken ahead was lost"

    # a caller that does not pass on what it was given: the step that ran ahead must not be used
    toks = random_tokens(V, 90, 77)
    ref = p.logits(toks)
    s = cache.alloc_slot()
    m.step(cache, [StepRequest(s, toks[:63], [])])
    before = runner.discarded
    for i in range(63, 90):                                # teacher forcing: the model's own pick is ignored
        runner.step_ids([s], [toks[i]], greedy, [0], [i])
        assert cache.length(s) == i + 1
    assert runner.discarded > before
    got_logits = m.step(cache, [StepRequest(s, [toks[0]], [0])])          # one more step reads the whole cache
    again = p.logits(toks + [toks[0]])
    assert_logits_close(got_logits.cpu(), again[-1:], dtype, "the cache after dropped steps")
    cache.free_slot(s)
    runner.drop_ahead()
    assert all(f == cache.n_pages for f in cache.free_pages())


def test_sampled_steps_inside_the_graph_follow_the_plain_sampler(folders):
    """Temperature, top-p and top-k sampling replayed inside the step's graph, seeds travelling with the descriptor:
    the same tokens as the plain sampler, request by request, while the batch shrinks."""
    import rocmforge_b200 as rf
    p = plain(folders, "B", "float32")
    llm = rf.LLM(folders("B", "float32"), dtype="float32")
    prompts = [random_tokens(384, n, 160 + n) for n in (3, 20, 41, 9)]
    for kw in (dict(temperature=0.8, top_p=1.0), dict(temperature=1.1, top_p=0.9, top_k=30)):
        out = llm.generate(prompts, max_tokens=25, seed=5, stop_token_ids=[7, 11, 13], **kw)
        for i, (pr, r) in enumerate(zip(prompts, out)):
            want, reason = S.generate(lambda t: p.logits(t)[-1].float(), pr, max_tokens=25, seed=5, request=i,
                                      stop_ids=(7, 11, 13), top_k=kw.get("top_k", 0), temperature=kw["temperature"],
                                      top_p=kw["top_p"])
            if r.tokens == want:
                assert r.reason == reason, f"request {i} with {kw}"
            else:
                check_sampled_up_to_swapped_neighbours(p, pr, r.tokens, want, kw["temperature"])
    assert llm.engine.decode_runner.launched_ahead > 0
    assert llm.cache.live_slots == 0 and all(f == llm.cache.n_pages for f in llm.cache.free_pages())
