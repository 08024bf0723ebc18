"""Decode steps replayed from CUDA graphs.

maeddesg/ROCmForge captures the tail of its decode step (norm, output matrix, argmax) as a HIP
graph and replays it per token (src/gpu/forward.rs:474-571); its full-step graph reads
position and length from a two-int device buffer uploaded before each replay
(src/gpu/cache.rs:707-734) but is switched off for a driver fault (forward.rs:2258-2275).
Here the whole step of a batch of B single tokens is one graph per B: token ids, slots and
positions live in a device descriptor that is rewritten before each replay, block tables
are read from the cache's device tables, so the graph's launches never change.
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch

import numpy as np

from ..cache import CacheError
from .batch import BatchError, DeviceDescriptor, StepBatch, StepRequest
from .context import StepContext


class _Captured:
    def __init__(self, graph, logits):
        self.graph = graph
        self.logits = logits


class DecodeRunner:
    """Runs one-token-per-sequence steps of a model over one cache from CUDA graphs: ``logits`` (a graph per batch size
    and context bucket, logits back), ``greedy_loop`` (ids fed back on the device, no host work between steps) and
    ``step_ids`` (sampler inside the graph, one step ahead of the host: what the generation loop uses)."""

    def __init__(self, model, cache, max_batch: int = 1024):
        self.model = model
        self.cache = cache
        # sized for the largest packed decode batch (tile tables included) and never moved: graphs keep its address
        self.desc = DeviceDescriptor(model.device, fixed=True, capacity=self.descriptor_words(max_batch))
        self.max_batch = max_batch
        self.graphs: Dict[tuple, _Captured] = {}
        self.replays = 0
        self._ready = None             # (slots, starts, packed descriptor without token ids, longest, cache epoch) of the next step
        self._flight = None            # a step launched before the host saw the ids of the step before it (see step_ids)
        self._templates: Dict[tuple, np.ndarray] = {}
        self._host_ids = []            # pinned buffers for sampled ids, used in turn
        self._turn = 0
        self.launched_ahead = 0        # steps that were launched ahead and served a call
        self.discarded = 0             # ... and that no call asked for

    @staticmethod
    def descriptor_words(max_batch: int) -> int:
        """int32 words of the largest packed decode descriptor (one token and one wanted row per sequence, seeds and
        row map of steps launched ahead)."""
        return StepBatch.layout(max_batch, max_batch, max_batch, decode_extras=True)[1]

    @staticmethod
    def length_bucket(longest: int) -> int:
        """Sequence-length bound a graph is captured for: the next power of two (at least 512).  Kernels
        whose launch shape grows with the context get this bound, so a graph serves until a sequence
        outgrows it; then the next bucket's graph is captured."""
        b = 512
        while b < longest:
            b *= 2
        return b

    def _context(self, B: int, bound: int) -> StepContext:
        views = self.desc.views(B, B, B)
        ctx = StepContext(self.model, views, T=B, B=B, R=B, is_decode=True, max_new=1,
                          max_end=min(bound, self.cache.max_seq_len))
        ctx.replayed = True          # launch shapes must not depend on this step's lengths
        return ctx

    def _warm_up(self, body) -> None:
        """Run ``body`` once outside capture (loads modules, sizes the allocator) and undo what it did to per-sequence
        state: the step it ran is not one of the sequence's steps."""
        saved = self.cache.snapshot_states()
        side = torch.cuda.Stream(device=self.model.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            body()
        torch.cuda.current_stream().wait_stream(side)
        self.cache.restore_states(saved)

    def _capture(self, B: int, bound: int, greedy: bool = False) -> _Captured:
        """The step's graph; with ``greedy`` the argmax is part of it and ``ids`` holds its result."""
        from .. import kernels
        ctx = self._context(B, bound)
        self._warm_up(lambda: self.model.forward(ctx, self.cache))
        graph = torch.cuda.CUDAGraph()
        ids = torch.zeros((B,), dtype=torch.int32, device=self.model.device) if greedy else None
        with torch.cuda.graph(graph):
            logits = self.model.forward(ctx, self.cache)
            if greedy:
                kernels.argmax(logits, out=ids)
        cap = _Captured(graph, logits)
        cap.ids = ids
        return cap

    def logits(self, slots: Sequence[int], tokens: Sequence[int], greedy: bool = False) -> torch.Tensor:
        """Step one token per slot; float32 logits [B, vocab] (a buffer reused by the next call), or with
        ``greedy`` the int32 ids [B] that the argmax inside the graph picked.

        The host's part of a step is split in two.  What does not depend on the new token ids (pages for the
        next position, the descriptor with every position moved on by one) is prepared right after the step's
        launch, while the device is busy; when the caller comes back with the sampled ids only those are
        filled in, copied and the graph replayed.  If the batch has changed meanwhile the prepared part is
        dropped and built afresh.
        """
        B = len(slots)
        if B > self.max_batch:
            raise ValueError(f"a decode batch of {B} exceeds the runner's limit of {self.max_batch}")
        slots = [int(s) for s in slots]
        starts = [self.cache.length(s) for s in slots]
        ready = self._ready
        self._ready = None
        # what was prepared ahead holds only while no slot was handed out or given back since: a slot that was
        # freed and filled again has the same number and may have the same length, but other pages
        if ready is not None and ready[4] == self.cache.epoch and ready[0] == slots and ready[1] == starts:
            packed, longest = ready[2], ready[3]
            toks = np.asarray(tokens, dtype=np.int64)
            if ((toks < 0) | (toks >= self.model.spec.vocab_size)).any():
                raise BatchError("a token id is outside the vocabulary")
            packed[:B] = toks
        else:
            requests = [StepRequest(s, [int(t)], [0]) for s, t in zip(slots, tokens)]
            batch = StepBatch(requests, starts, self.model.spec.vocab_size)
            self.cache.prepare(slots, [1] * B)
            packed, longest = batch.pack(), max(starts) + 1
        self.desc.upload(packed)
        key = (B, self.length_bucket(longest), greedy)
        cap = self.graphs.get(key)
        if cap is None:
            cap = self.graphs[key] = self._capture(B, key[1], greedy)
        cap.graph.replay()
        self.replays += 1
        self.cache.commit(slots, [1] * B)
        # while the device works: the next step of the same batch, all but its token ids
        try:
            self.cache.prepare(slots, [1] * B)
            lay, _ = StepBatch.layout(B, B, B)
            nxt = packed.copy()
            for name in ("tok_pos", "seq_start"):
                o, n = lay[name]
                nxt[o:o + n] += 1
            self._ready = (slots, [x + 1 for x in starts], nxt, longest + 1, self.cache.epoch)
        except CacheError:
            self._ready = None                     # no room for a further token: the next call will say so if it comes
        return cap.ids if greedy else cap.logits

    # ---------------------------------------------------------------- replay without host work
    def greedy_loop(self, slots: Sequence[int], tokens: Sequence[int], steps: int):
        """``steps`` greedy decode steps whose sampled ids feed the next step on the device.

        Returns (ids [steps, B] int32 on the device, start event, end event, launches per step).
        Pages for all steps are taken first, so the loop itself is nothing but graph replays.
        """
        from .. import kernels
        B = len(slots)
        self._ready = None
        self.cache.reserve(slots, [self.cache.length(s) + steps for s in slots])
        requests = [StepRequest(s, [int(t)], [0]) for s, t in zip(slots, tokens)]
        batch = StepBatch(requests, [self.cache.length(s) for s in slots], self.model.spec.vocab_size)
        self.desc.upload(batch.pack())
        bound = self.length_bucket(max(self.cache.length(s) for s in slots) + steps)
        key = ("loop", B, bound)
        out = torch.empty((steps, B), dtype=torch.int32, device=self.model.device)
        cap = self.graphs.get(key)
        if cap is None:
            ctx = self._context(B, bound)
            sampled = torch.zeros((B,), dtype=torch.int32, device=self.model.device)
            self._warm_up(lambda: kernels.argmax(self.model.forward(ctx, self.cache), out=sampled))
            graph = torch.cuda.CUDAGraph()
            n0 = kernels.launch_count()
            with torch.cuda.graph(graph):
                kernels.argmax(self.model.forward(ctx, self.cache), out=sampled)
                kernels.advance_decode(ctx.tokens, ctx.tok_pos, ctx.seq_start, sampled)
            cap = self.graphs[key] = _Captured(graph, sampled)
            cap.launches = kernels.launch_count() - n0
            self.desc.upload(batch.pack())          # warm-up and capture did not advance anything, but be exact
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            cap.graph.replay()
            out[i].copy_(cap.logits, non_blocking=True)
        end.record()
        self.replays += steps
        self.cache.commit(slots, [steps] * B)
        return out, start, end, cap.launches

    # ---------------------------------------------------------------- sampled ids, one step ahead of the host
    def _capture_ids(self, B: int, bound: int, sampling) -> _Captured:
        """The step's graph with the sampler inside: forward, then argmax or the seeded draw (seeds from the descriptor)."""
        from .. import kernels
        ctx = self._context(B, bound)
        seeds = self.desc.views(B, B, B, decode_extras=True)["seeds"].view(torch.int64)
        ids = torch.zeros((B,), dtype=torch.int32, device=self.model.device)

        def body():
            logits = self.model.forward(ctx, self.cache)
            if sampling.greedy:
                kernels.argmax(logits, out=ids)
            else:
                kernels.sample(logits, sampling.temperature, sampling.top_p, sampling.top_k, seeds, out=ids)
            return logits
        self._warm_up(body)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = body()
        cap = _Captured(graph, logits)
        cap.ids = ids
        return cap

    def _pinned(self, B: int):
        if not self._host_ids:
            for _ in range(3):
                t = torch.empty((self.max_batch,), dtype=torch.int32).pin_memory()
                self._host_ids.append((t, t.numpy(), torch.cuda.Event()))
        self._turn = (self._turn + 1) % len(self._host_ids)
        return self._host_ids[self._turn]

    def _launch(self, slots, starts, sampling, requests, draws, tokens=None, ids_from=None, row_map=None):
        """Enqueue one decode step of ``slots`` at positions ``starts``: descriptor upload, the tokens (from the host, or
        gathered on the device from the ids of the step before), graph replay, copy of the sampled ids to pinned memory."""
        from .. import kernels
        from ..sampling.params import as_int64, draw_seed
        B = len(slots)
        key = tuple(slots)
        lay, total = StepBatch.layout(B, B, B, decode_extras=True)
        packed = self._templates.get(key)
        if packed is None:
            if len(self._templates) > 256:
                self._templates.clear()
            packed = np.zeros((total,), dtype=np.int32)
            for name, arr in (("tok_seq", np.arange(B)), ("seq_slot", np.asarray(slots)), ("seq_nnew", np.ones(B)),
                              ("cu_q", np.arange(B + 1)), ("want_rows", np.arange(B))):
                o, n = lay[name]
                packed[o:o + n] = arr
            self._templates[key] = packed
        for name in ("tok_pos", "seq_start"):
            o, n = lay[name]
            packed[o:o + n] = starts
        if tokens is not None:
            packed[:B] = tokens
        if not sampling.greedy:
            o, n = lay["seeds"]
            packed[o:o + n].view(np.int64)[:] = [as_int64(draw_seed(sampling.seed, r, d)) for r, d in zip(requests, draws)]
        if row_map is not None:
            o, n = lay["row_map"]
            packed[o:o + n] = row_map
        self.desc.upload(packed)
        if tokens is None:
            views = self.desc.views(B, B, B, decode_extras=True)
            kernels.gather_tokens(views["tokens"], ids_from, views["row_map"])
        gkey = ("ids", B, self.length_bucket(max(starts) + 1), sampling.greedy,
                None if sampling.greedy else (sampling.temperature, sampling.top_p, sampling.top_k))
        cap = self.graphs.get(gkey)
        if cap is None:
            cap = self.graphs[gkey] = self._capture_ids(B, gkey[2], sampling)
            self.desc.upload(packed)                       # capture ran the step: put the descriptor back as it was
            if tokens is None:
                kernels.gather_tokens(views["tokens"], ids_from, views["row_map"])
        cap.graph.replay()
        self.replays += 1
        pinned, host, event = self._pinned(B)
        pinned[:B].copy_(cap.ids, non_blocking=True)
        event.record()
        return dict(slots=list(slots), gens=[self.cache.generation(s) for s in slots], starts=list(starts), cap=cap,
                    host=host, event=event, sampling=sampling, requests=list(requests), draws=list(draws), B=B)

    def step_ids(self, slots: Sequence[int], tokens: Sequence[int], sampling, requests: Sequence[int],
                 draws: Sequence[int], more: bool = True):
        """Step one token per slot and sample the next; returns the sampled ids as a list.

        The device runs one step ahead of the host.  Before this call waits for its own ids it launches the next
        step of the same sequences, whose tokens the device takes from this step's ids itself (``more`` = the
        caller will come back unless sequences stop).  The next call then finds its step already running: it
        checks that the caller passes the ids it was given, waits and returns.  Sequences that ended in between
        are simply left out (their rows of the step that ran ahead are ignored, the rows of the others are as
        valid as ever: a row does not depend on its neighbours).  If the call asks for anything else (other
        tokens, other sequences, other sampling) the step that ran ahead is dropped and its pages given back.
        """
        slots = [int(s) for s in slots]
        B = len(slots)
        if B > self.max_batch:
            raise ValueError(f"a decode batch of {B} exceeds the runner's limit of {self.max_batch}")
        self._ready = None
        cache = self.cache
        fl, self._flight = self._flight, None
        rows = None
        if fl is not None:
            where = {s: i for i, s in enumerate(fl["slots"])}
            rows = [where.get(s, -1) for s in slots]
            fits = (fl["sampling"] == sampling and all(r >= 0 for r in rows)
                    and all(cache.slots.is_held(s) and cache.generation(s) == fl["gens"][r] and cache.length(s) == fl["starts"][r]
                            and int(t) == fl["fed"][r] and rq == fl["requests"][r] and d == fl["draws"][r]
                            for s, r, t, rq, d in zip(slots, rows, tokens, requests, draws)))
            if not fits:
                self.discarded += 1
                cache.rollback([s for s, g in zip(fl["slots"], fl["gens"])
                                if cache.slots.is_held(s) and cache.generation(s) == g])
                fl = rows = None
        if fl is None:
            toks = np.asarray(tokens, dtype=np.int64)
            if ((toks < 0) | (toks >= self.model.spec.vocab_size)).any():
                raise BatchError("a token id is outside the vocabulary")
            starts = [cache.length(s) for s in slots]
            cache.prepare(slots, [1] * B)
            try:
                fl = self._launch(slots, starts, sampling, requests, draws, tokens=toks)
            except BaseException:
                cache.rollback(slots)
                raise
            rows = list(range(B))
        else:
            self.launched_ahead += 1
        cache.commit(slots, [1] * B)                       # the step is under way for these sequences
        if more and not cache.states:
            # (a model with per-sequence state is not run ahead: a step that is dropped would have changed the state,
            # whereas keys and values written by a dropped step are simply written again)
            # the next step of the same sequences, before the host knows this step's ids
            try:
                cache.prepare(slots, [1] * B)
            except CacheError:
                pass                                       # no room for a further token: the caller will learn it if it comes back
            else:
                try:
                    self._flight = self._launch(slots, [cache.length(s) for s in slots], sampling, requests,
                                                [d + 1 for d in draws], ids_from=fl["cap"].ids, row_map=rows)
                except BaseException:
                    cache.rollback(slots)
                    raise
        fl["event"].synchronize()
        got = fl["host"][:fl["B"]].tolist()
        ids = [got[r] for r in rows]
        if self._flight is not None:
            self._flight["fed"] = ids                      # what the step that runs ahead was fed, row by row
        return ids

    def drop_ahead(self) -> None:
        """Forget a step that was launched ahead (its pages go back); the device finishes it unobserved."""
        fl, self._flight = self._flight, None
        if fl is not None:
            self.discarded += 1
            self.cache.rollback([s for s, g in zip(fl["slots"], fl["gens"])
                                 if self.cache.slots.is_held(s) and self.cache.generation(s) == g])
