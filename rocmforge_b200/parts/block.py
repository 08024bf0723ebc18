"""Arrangements of parts around the residual stream."""
from __future__ import annotations

from typing import Dict

from .base import BLOCKS, Block, FeedForward, Mixer, Norm, Part


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x))
    (maeddesg/ROCmForge src/gpu/forward.rs:930-1161; src/cpu/forward.rs:18-337).

    ``names`` maps the four parts to their prefixes inside the layer, as the
    architecture's tensor names have them.
    """

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward, names: Dict[str, str]):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.names = dict(names)

    def sub_parts(self) -> Dict[str, Part]:
        return {self.names["norm1"]: self.norm1, self.names["mixer"]: self.mixer,
                self.names["norm2"]: self.norm2, self.names["ffn"]: self.ffn}

    def entry_norm(self):
        return self.norm1 if self.mixer.accepts_scaled_rows else None

    def forward(self, ctx, stream, cache_view):
        after = stream.after_block                   # the norm that follows this block (the model knows the order)
        y = self.norm1.forward(ctx, stream, deferred_ok=self.mixer.accepts_scaled_rows)
        stream.next_norm = self.norm2 if self.ffn.accepts_scaled_rows else None
        self.mixer.forward(ctx, y, cache_view, stream)
        y = self.norm2.forward(ctx, stream, deferred_ok=self.ffn.accepts_scaled_rows)
        stream.next_norm = after
        self.ffn.forward(ctx, y, stream)
        stream.next_norm = None
