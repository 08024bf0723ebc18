"""The replayed decode paths of ``DecodeRunner`` against the plain model (needs a GPU): the loop that feeds the
sampled ids back on the device, and the step that is prepared ahead of time while slots come and go."""
import pytest
import torch

from helpers import CONFIGS, assert_logits_close, random_tokens
from plain import sampling_plain as S
from test_engine_gpu import check_tokens_up_to_near_ties, engine, plain, poison_free_pages

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
