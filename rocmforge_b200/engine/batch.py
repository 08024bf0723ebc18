"""A step's batch: which sequences bring which tokens, and where logits are wanted.

maeddesg/ROCmForge runs one sequence: ``gpu_prefill_forward_hybrid(tokens, start_pos=0)`` for a
whole prompt (src/gpu/forward.rs:1198) and ``gpu_full_forward_hybrid(pos)`` for one token
(:2589), with the logits of the last row only (:256-264).  Here one descriptor covers a
ragged batch of both: tokens of all sequences are concatenated (no padding rows), each
token knows its sequence and absolute position, and logits are produced for the rows
that were asked for.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch


class BatchError(ValueError):
    pass


@dataclass
class StepRequest:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()          # indices among ``tokens`` whose logits are wanted


class StepBatch:
    """Host side of a step: flat int32 arrays, packed into one buffer for a single copy.

    ``tables``: further int32 arrays that parts of the model build on the host for their kernels from this batch
    ({name: function of the batch}); they travel in the same copy and appear as ``StepContext.tables[name]``."""

    def __init__(self, requests: Sequence[StepRequest], starts: Sequence[int], vocab_size: int, tables=None):
        if not requests:
            raise BatchError("a step needs at least one sequence")
        self.slots = [int(r.slot) for r in requests]
        self.n_new = np.array([len(r.tokens) for r in requests], dtype=np.int32)
        if (self.n_new <= 0).any():
            raise BatchError("every sequence of a step must bring at least one token")
        self.starts = np.asarray(starts, dtype=np.int32)
        self.B = len(requests)
        self.T = int(self.n_new.sum())
        self.cu_q = np.zeros((self.B + 1,), dtype=np.int32)
        np.cumsum(self.n_new, out=self.cu_q[1:])
        self.tokens = np.concatenate([np.asarray(r.tokens, dtype=np.int64) for r in requests])
        bad = np.nonzero((self.tokens < 0) | (self.tokens >= vocab_size))[0]
        if len(bad):
            # the reference checks ids before its gather, src/gpu/forward.rs:834-842
            raise BatchError(f"token id {int(self.tokens[bad[0]])} is outside the vocabulary of {vocab_size}")
        self.tokens = self.tokens.astype(np.int32)
        self.tok_seq = np.repeat(np.arange(self.B, dtype=np.int32), self.n_new)
        self.tok_pos = (np.arange(self.T, dtype=np.int32) - self.cu_q[:-1][self.tok_seq]
                        + self.starts[self.tok_seq]).astype(np.int32)
        rows: List[int] = []
        for i, r in enumerate(requests):
            for w in r.want:
                if not 0 <= int(w) < len(r.tokens):
                    raise BatchError(f"slot {r.slot}: logits wanted at place {w} of {len(r.tokens)} tokens")
                rows.append(int(self.cu_q[i]) + int(w))
        self.want_rows = np.asarray(rows, dtype=np.int32)
        self.R = len(rows)
        self.is_decode = bool((self.n_new == 1).all())
        self.max_new = int(self.n_new.max())
        self.max_end = int((self.starts + self.n_new).max())
        self.tables = {name: np.ascontiguousarray(build(self), dtype=np.int32).reshape(-1)
                       for name, build in (tables or {}).items()}

    @property
    def extras(self):
        """(name, length) of the parts' tables, in packing order."""
        return tuple((name, int(arr.size)) for name, arr in self.tables.items())

    # layout of the packed descriptor, in int32 elements
    @staticmethod
    def layout(T: int, B: int, R: int, extras=(), decode_extras: bool = False):
        """``extras``: (name, length) of the parts' tables.  ``decode_extras``: two more arrays for decode steps that
        a runner launches ahead of the host: the rows' 64-bit sampling seeds (two words each) and each sequence's row
        in the step before."""
        names = [("tokens", T), ("tok_seq", T), ("tok_pos", T), ("seq_slot", B), ("seq_start", B),
                 ("seq_nnew", B), ("cu_q", B + 1), ("want_rows", R)] + [(n, k) for n, k in extras]
        if decode_extras:
            names += [("seeds", 2 * B), ("row_map", B)]
        off, out = 0, {}
        for name, n in names:
            out[name] = (off, n)
            off += (n + 3) // 4 * 4            # keep every array 16-byte aligned
        return out, off

    def pack(self) -> np.ndarray:
        lay, total = self.layout(self.T, self.B, self.R, self.extras)
        buf = np.zeros((total,), dtype=np.int32)
        for name, arr in [("tokens", self.tokens), ("tok_seq", self.tok_seq), ("tok_pos", self.tok_pos),
                          ("seq_slot", np.asarray(self.slots, dtype=np.int32)), ("seq_start", self.starts),
                          ("seq_nnew", self.n_new), ("cu_q", self.cu_q), ("want_rows", self.want_rows)] + list(self.tables.items()):
            o, n = lay[name]
            buf[o:o + n] = arr
        return buf


class DeviceDescriptor:
    """The device copy of a step descriptor, with one pinned staging buffer for the upload."""

    def __init__(self, device, capacity: int = 4096, fixed: bool = False):
        """``fixed``: the device buffer is never replaced (captured graphs hold views of it); a descriptor
        larger than ``capacity`` is then an error instead of a reason to grow."""
        self.device = torch.device(device)
        self.fixed = fixed
        self.capacity = 0
        self.dev: Optional[torch.Tensor] = None
        self.pinned: Optional[torch.Tensor] = None
        self._done: Optional[torch.cuda.Event] = None
        self._grow(capacity)

    def _grow(self, n: int) -> None:
        if self._done is not None:
            self._done.synchronize()
        self.capacity = n
        self.dev = torch.zeros((n,), dtype=torch.int32, device=self.device)
        self.pinned = torch.zeros((n,), dtype=torch.int32)
        if self.device.type == "cuda":
            self.pinned = self.pinned.pin_memory()
            if self._done is None:
                self._done = torch.cuda.Event()
        self._pinned_np = self.pinned.numpy()          # the same memory, written without a tensor per call
        self._slices = {}                              # n -> (device slice, pinned slice)
        self._busy = False

    def upload(self, packed: np.ndarray) -> None:
        """One copy of the packed descriptor to the device, on the current stream.  This sits between a step's
        result and the next step's launch, so it does as little on the host as it can."""
        n = packed.shape[0]
        if n > self.capacity:
            if self.fixed:
                raise BatchError(f"a step descriptor of {n} words does not fit the {self.capacity} this runner "
                                 "was sized for")
            self._grow(max(n, 2 * self.capacity))
        if self._busy:
            self._done.synchronize()               # the previous copy may still read the staging buffer
        self._pinned_np[:n] = packed
        pair = self._slices.get(n)
        if pair is None:
            pair = self._slices[n] = (self.dev[:n], self.pinned[:n])
        pair[0].copy_(pair[1], non_blocking=True)
        if self._done is not None:
            self._done.record()
            self._busy = True

    def views(self, T: int, B: int, R: int, extras=(), decode_extras: bool = False):
        lay, _ = StepBatch.layout(T, B, R, extras, decode_extras)
        return {name: self.dev[o:o + n] for name, (o, n) in lay.items()}
