"""The cache of a model: a slot for each live sequence, keys and values in pages, and
fixed-size per-sequence state beside them.

maeddesg/ROCmForge keeps one K and one V buffer of ``max_seq`` rows per layer for its single
sequence (src/gpu/cache.rs:23-83).  Here a sequence holds a *slot*; the slot owns pages of
64 positions, taken from a pool when the sequence grows and given back when it ends, so
the pool is sized by the tokens that live sequences hold together.  Layers whose needs
differ (all keys / a window of them / other head counts) form groups with storage, pool
and block table of their own; a group with a window drops the pages that have fallen
out of every future query's window.  Mixers that ask for a ``StateRequest`` get tensors
indexed by slot, zeroed when the slot is handed out.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .pages import CacheError, FreeList
from .requests import KVRequest, StateRequest

PAGE = 64


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


class KVGroup:
    """Pages, pool and block table shared by the cache owners with one KVRequest."""

    def __init__(self, request: KVRequest, owners: List[int], n_pages: int, max_slots: int,
                 max_pages_per_seq: int, dtype: torch.dtype, device):
        self.request = request
        self.owners = list(owners)
        self.index_of = {o: i for i, o in enumerate(self.owners)}
        self.n_pages = n_pages
        self.max_pages_per_seq = max_pages_per_seq
        self.window = request.window
        self.pool = FreeList(n_pages, "cache page")
        # [owner, k|v, page, kv_head, position in page, head_dim]
        self.storage = torch.zeros((len(self.owners), 2, n_pages, request.n_kv_heads, PAGE, request.head_dim),
                                   dtype=dtype, device=device)
        self.table = np.full((max_slots, max_pages_per_seq), -1, dtype=np.int32)
        self.table_dev = torch.zeros((max_slots, max_pages_per_seq), dtype=torch.int32, device=device)
        self._dirty: Dict[int, List[int]] = {}          # slot -> [lo, hi) of changed entries
        self._upload_done: Optional[torch.cuda.Event] = None
        self._staging: Optional[torch.Tensor] = None

    # --- pages of one slot
    def first_needed_page(self, length_after: int) -> int:
        """Lowest logical page any query at position >= length_after - 1 ... can still see."""
        if self.window is None:
            return 0
        # the next query (position length_after) sees keys >= length_after - window + 1
        lo = length_after - self.window + 1
        return max(lo, 0) // PAGE

    def pages_missing(self, slot: int, start: int, end: int) -> int:
        """Pages to be taken so that positions [start, end) can be written and read."""
        lo = 0 if self.window is None else max(start - self.window + 1, 0)
        need = 0
        for p in range(lo // PAGE, pages_for(end)):
            if self.table[slot, p] < 0:
                need += 1
        return need

    def ensure(self, slot: int, start: int, end: int) -> None:
        if pages_for(end) > self.max_pages_per_seq:
            raise CacheError(f"a sequence of {end} tokens needs {pages_for(end)} pages; "
                             f"the block table holds {self.max_pages_per_seq} per sequence")
        for p in range(start // PAGE, pages_for(end)):
            if self.table[slot, p] < 0:
                self.table[slot, p] = self.pool.take()
                self._mark(slot, p)

    def trim(self, slot: int, length: int) -> None:
        """Give back pages no future query of this slot can see (window groups only)."""
        if self.window is None:
            return
        keep_from = self.first_needed_page(length)
        row = self.table[slot]
        for p in range(keep_from - 1, -1, -1):
            if row[p] < 0:
                break                                   # everything below was trimmed earlier
            self.pool.give_back(int(row[p]))
            row[p] = -1
            self._mark(slot, p)                         # the device table must not name a free page either

    def release(self, slot: int) -> None:
        row = self.table[slot]
        for p in np.nonzero(row >= 0)[0]:
            self.pool.give_back(int(row[p]))
            row[p] = -1
            self._mark(slot, int(p))                    # the next upload clears the device entry as well

    def drop_beyond(self, slot: int, length: int) -> None:
        """Give back the pages that lie wholly beyond ``length`` positions (taken for a step that did not happen)."""
        row = self.table[slot]
        for p in range(pages_for(length), self.max_pages_per_seq):
            if row[p] >= 0:
                self.pool.give_back(int(row[p]))
                row[p] = -1
                self._mark(slot, p)

    def held_pages(self, slot: int) -> List[int]:
        row = self.table[slot]
        return [int(x) for x in row[row >= 0]]

    def _mark(self, slot: int, p: int) -> None:
        r = self._dirty.get(slot)
        if r is None:
            self._dirty[slot] = [p, p + 1]
        else:
            r[0] = min(r[0], p)
            r[1] = max(r[1], p + 1)

    def upload(self) -> None:
        """Copy the changed block-table entries to the device, on the current stream."""
        if not self._dirty:
            return
        if self.table_dev.is_cuda:
            n = sum(hi - lo for lo, hi in self._dirty.values())
            if self._upload_done is not None:
                self._upload_done.synchronize()         # the staging buffer may still be read
            if self._staging is None or self._staging.numel() < n:
                self._staging = torch.empty((max(n, 1024),), dtype=torch.int32).pin_memory()
            off = 0
            for slot, (lo, hi) in self._dirty.items():
                k = hi - lo
                self._staging[off:off + k] = torch.from_numpy(self.table[slot, lo:hi])
                self.table_dev[slot, lo:hi].copy_(self._staging[off:off + k], non_blocking=True)
                off += k
            self._upload_done = torch.cuda.Event()
            self._upload_done.record()
        else:
            for slot, (lo, hi) in self._dirty.items():
                self.table_dev[slot, lo:hi] = torch.from_numpy(self.table[slot, lo:hi].copy())
        self._dirty.clear()

    def k_pages(self, owner: int) -> torch.Tensor:
        return self.storage[self.index_of[owner], 0]

    def v_pages(self, owner: int) -> torch.Tensor:
        return self.storage[self.index_of[owner], 1]


@dataclass
class KVView:
    """What an attention-like mixer sees of its layer's cache."""
    k_pages: torch.Tensor           # [n_pages, kv_heads, 64, head_dim]
    v_pages: torch.Tensor
    block_table: torch.Tensor       # [max_slots, max_pages_per_seq] int32 on the device
    window: Optional[int]
    writes: bool                    # False: this layer only reads another layer's keys and values


@dataclass
class StateView:
    """Fixed-size state tensors of a mixer, each [max_slots, *shape]."""
    tensors: Dict[str, torch.Tensor]

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.tensors[name]


class SequenceCache:
    """Slots, page groups and state for one model instance.

    ``requests`` maps a cache owner (an index into the model's schedule) to what its mixer
    asked for.  ``max_tokens`` is the number of positions live sequences may hold together,
    each sequence rounded up to whole pages.
    """

    def __init__(self, requests: Dict[int, object], *, max_tokens: int, max_slots: Optional[int] = None,
                 max_seq_len: Optional[int] = None, dtype: torch.dtype = torch.float32, device="cpu"):
        if max_tokens <= 0:
            raise CacheError("max_tokens must be positive")
        self.device = torch.device(device)
        self.dtype = dtype
        self.n_pages = pages_for(max_tokens)
        self.max_slots = int(max_slots) if max_slots else min(self.n_pages, 4096)
        per_seq = self.n_pages if not max_seq_len else min(self.n_pages, pages_for(max_seq_len))
        self.max_pages_per_seq = max(per_seq, 1)
        self.max_seq_len = self.max_pages_per_seq * PAGE if not max_seq_len else min(max_seq_len, self.max_pages_per_seq * PAGE)
        self.slots = FreeList(self.max_slots, "slot")
        self.lengths = np.zeros((self.max_slots,), dtype=np.int64)
        # grows whenever a slot is handed out or given back: whoever prepared a step ahead of time (pages taken,
        # descriptor built) compares it and drops what it prepared when the set of sequences has changed
        self.epoch = 0
        self.generations = np.zeros((self.max_slots,), dtype=np.int64)      # how often each slot was handed out

        by_key: Dict[tuple, List[int]] = {}
        self._kv_request: Dict[tuple, KVRequest] = {}
        self.states: Dict[int, StateView] = {}
        for owner in sorted(requests):
            req = requests[owner]
            if req is None:
                continue
            if isinstance(req, KVRequest):
                by_key.setdefault(req.group_key(), []).append(owner)
                self._kv_request[req.group_key()] = req
            elif isinstance(req, StateRequest):
                tensors = {}
                for name, shape, dt in req.tensors:
                    tensors[name] = torch.zeros((self.max_slots, *shape), dtype=dt or dtype, device=self.device)
                self.states[owner] = StateView(tensors)
            else:
                raise CacheError(f"cache owner {owner}: unknown kind of request {req!r}")
        self.groups: List[KVGroup] = [
            KVGroup(self._kv_request[key], owners, self.n_pages, self.max_slots, self.max_pages_per_seq,
                    dtype, self.device) for key, owners in by_key.items()]
        self._group_of: Dict[int, KVGroup] = {o: g for g in self.groups for o in g.owners}

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        slot = self.slots.take()
        self.epoch += 1
        self.generations[slot] += 1
        self.lengths[slot] = 0
        for view in self.states.values():
            for t in view.tensors.values():
                t[slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is freed but not held")
        for g in self.groups:
            g.release(slot)
        self.lengths[slot] = 0
        self.slots.give_back(slot)
        self.epoch += 1

    def generation(self, slot: int) -> int:
        """Which holder of the slot this is (it grows when the slot is handed out): a step prepared for a slot belongs
        to one holder, and the number of a freed slot comes back with the next sequence."""
        return int(self.generations[slot])

    def length(self, slot: int) -> int:
        return int(self.lengths[slot])

    @property
    def live_slots(self) -> int:
        return self.slots.n_held

    def free_pages(self) -> List[int]:
        return [g.pool.n_free for g in self.groups]

    # ------------------------------------------------------------------ steps
    def prepare(self, slots: Sequence[int], n_new: Sequence[int]) -> np.ndarray:
        """Make room for ``n_new[i]`` more tokens in ``slots[i]``; returns each start position.

        Nothing is taken if the step as a whole does not fit.
        """
        if len(set(slots)) != len(slots):
            raise CacheError(f"a slot appears twice in one step: {list(slots)}")
        starts = np.zeros((len(slots),), dtype=np.int64)
        for i, (s, n) in enumerate(zip(slots, n_new)):
            if not self.slots.is_held(s):
                raise CacheError(f"slot {s} is not held by any sequence")
            if n <= 0:
                raise CacheError(f"slot {s}: a step must bring at least one token")
            starts[i] = self.lengths[s]
            if starts[i] + n > self.max_seq_len:
                raise CacheError(f"slot {s}: {starts[i]} cached + {n} new tokens exceed the longest "
                                 f"sequence the cache holds ({self.max_seq_len})")
        for g in self.groups:
            need = sum(g.pages_missing(s, int(st), int(st + n)) for s, st, n in zip(slots, starts, n_new))
            if need > g.pool.n_free:
                raise CacheError(f"the step needs {need} more cache pages, {g.pool.n_free} of "
                                 f"{g.n_pages} are free (raise max_tokens or end sequences)")
        for g in self.groups:
            for s, st, n in zip(slots, starts, n_new):
                g.ensure(s, int(st), int(st + n))
            g.upload()
        return starts

    def reserve(self, slots: Sequence[int], upto_len: Sequence[int]) -> None:
        """Take the pages for positions < upto_len[i] of slots[i] now (steps replayed without host work need
        them).  Nothing is taken if not all of it fits."""
        for s, n in zip(slots, upto_len):
            if not self.slots.is_held(s):
                raise CacheError(f"slot {s} is not held by any sequence")
            if n > self.max_seq_len:
                raise CacheError(f"slot {s}: {n} tokens exceed the longest sequence the cache holds "
                                 f"({self.max_seq_len})")
        for g in self.groups:
            need = sum(g.pages_missing(s, int(self.lengths[s]), int(n)) for s, n in zip(slots, upto_len))
            if need > g.pool.n_free:
                raise CacheError(f"reserving needs {need} more cache pages, {g.pool.n_free} of {g.n_pages} are free")
        for g in self.groups:
            for s, n in zip(slots, upto_len):
                g.ensure(s, int(self.lengths[s]), int(n))
            g.upload()

    def rollback(self, slots: Sequence[int]) -> None:
        """Undo ``prepare``/``reserve`` for a step that failed: every slot keeps the pages of its committed length only."""
        for s in slots:
            if self.slots.is_held(s):
                for g in self.groups:
                    g.drop_beyond(s, int(self.lengths[s]))

    def commit(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        for s, n in zip(slots, n_new):
            self.lengths[s] += n
            for g in self.groups:
                g.trim(s, int(self.lengths[s]))

    # ------------------------------------------------------------------ views
    def kv_view(self, owner: int, writes: bool = True) -> KVView:
        g = self._group_of[owner]
        return KVView(g.k_pages(owner), g.v_pages(owner), g.table_dev, g.window, writes)

    def state_view(self, owner: int) -> StateView:
        return self.states[owner]

    def view(self, owner: int, writes: bool = True):
        if owner in self._group_of:
            return self.kv_view(owner, writes)
        if owner in self.states:
            return self.states[owner]
        return None

    def snapshot_states(self):
        """Copies of every fixed-size state tensor (for a step that is run once without being meant: unlike keys and
        values, which a repeated step writes again with the same contents, state is read, changed and written)."""
        return [(t, t.clone()) for v in self.states.values() for t in v.tensors.values()]

    @staticmethod
    def restore_states(snapshot) -> None:
        for t, saved in snapshot:
            t.copy_(saved)

    def memory_bytes(self) -> int:
        n = sum(g.storage.numel() * g.storage.element_size() for g in self.groups)
        n += sum(t.numel() * t.element_size() for v in self.states.values() for t in v.tensors.values())
        return n
