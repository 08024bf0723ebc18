"""The generation loop above the step function.

maeddesg/ROCmForge's loop (src/main.rs:911-983; chat variant src/cli/chat.rs:538-613) serves one
sequence: sample the first token from the prompt's logits, then repeat {stop?, emit,
forward, sample}.  This loop does the same for batches of unequal prompts that start
together: all prompts in one step, then one token for each sequence that still runs;
a sequence that ends leaves the batch and its slot is given back at once; when more
requests are waiting than fit, batches follow one another.

The loop itself only decides; everything that touches the device sits behind a small
``StepEngine`` face, so that the decisions can be tested without one.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, List, Optional, Sequence

from ..sampling.params import SamplingParams

# reasons a sequence ends with (the reference's chat loop reports EOS / max tokens / ctx full,
# src/cli/chat.rs:703-722)
STOP_TOKEN = "stop_token"
MAX_TOKENS = "max_tokens"
CONTEXT_FULL = "context_full"


@dataclass
class GenerationResult:
    prompt_len: int
    tokens: List[int] = field(default_factory=list)
    reason: str = ""


class StepEngine:
    """What the loop needs from below."""

    max_seq_len: int

    def admit(self, prompt_lens: Sequence[int], max_new_tokens: int) -> int:
        """How many of the waiting requests (in order, at least one if any can ever fit) form the next batch."""
        raise NotImplementedError

    def alloc_slot(self) -> int:
        raise NotImplementedError

    def free_slot(self, slot: int) -> None:
        raise NotImplementedError

    wants_final_hint = False

    def run(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], requests: Sequence[int],
            draws: Sequence[int], sampling: SamplingParams) -> List[int]:
        """Step the given tokens of each slot and sample one next token per slot.

        An engine that sets ``wants_final_hint`` also gets ``final=`` (the tokens sampled by this call are the last
        ones of all its sequences whatever they are): it may then spare itself work it would do ahead of time."""
        raise NotImplementedError


def generate(engine: StepEngine, prompts: Sequence[Sequence[int]], *, max_new_tokens: int,
             sampling: Optional[SamplingParams] = None, stop_token_ids: Iterable[int] = (),
             on_token=None) -> List[GenerationResult]:
    """Generate up to ``max_new_tokens`` tokens for every prompt.

    A stop token ends its sequence and is not part of the output (src/main.rs:913-923).
    ``on_token(request index, token)`` is called for every emitted token.
    """
    sampling = sampling or SamplingParams()
    stop = set(int(t) for t in stop_token_ids)
    results = [GenerationResult(prompt_len=len(p)) for p in prompts]
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"request {i}: the prompt is empty")          # src/gpu/forward.rs:1211
        if len(p) > engine.max_seq_len:
            raise ValueError(f"request {i}: the prompt has {len(p)} tokens, the cache holds "
                             f"{engine.max_seq_len} per sequence")         # src/gpu/forward.rs:1224-1232
    if max_new_tokens <= 0:
        for r in results:
            r.reason = MAX_TOKENS
        return results

    waiting = list(range(len(prompts)))
    while waiting:
        n = engine.admit([len(prompts[i]) for i in waiting], max_new_tokens)
        if n <= 0:
            raise RuntimeError(f"request {waiting[0]} does not fit into the cache even alone")
        batch, waiting = waiting[:n], waiting[n:]
        _run_batch(engine, batch, prompts, results, max_new_tokens, sampling, stop, on_token)
    return results


def _run_batch(engine, batch, prompts, results, max_new_tokens, sampling, stop, on_token) -> None:
    slot = {i: engine.alloc_slot() for i in batch}
    try:
        pos = {i: len(prompts[i]) for i in batch}          # position the next emitted token will take
        draws = {i: 0 for i in batch}
        active = list(batch)
        nxt = engine.run([slot[i] for i in active], [prompts[i] for i in active], active,
                         [draws[i] for i in active], sampling)
        while True:
            still, feed = [], []
            for i, tok in zip(active, nxt):
                draws[i] += 1
                r = results[i]
                # order of the checks as in src/main.rs:913
                if tok in stop:
                    r.reason = STOP_TOKEN
                elif pos[i] >= engine.max_seq_len:
                    r.reason = CONTEXT_FULL
                else:
                    r.tokens.append(int(tok))
                    if on_token is not None:
                        on_token(i, int(tok))
                    if len(r.tokens) >= max_new_tokens:
                        r.reason = MAX_TOKENS       # the last token need not be run through the model
                    else:
                        still.append(i)
                        feed.append([int(tok)])
                        continue
                engine.free_slot(slot.pop(i))       # a sequence that ended gives its slot back at once
            if not still:
                return
            active = still
            hint = {}
            if engine.wants_final_hint:
                hint["final"] = all(len(results[i].tokens) + 1 >= max_new_tokens for i in active)
            nxt = engine.run([slot[i] for i in active], feed, active, [draws[i] for i in active], sampling, **hint)
            for i in active:
                pos[i] += 1
    finally:
        for s in slot.values():
            engine.free_slot(s)
