"""Additions to the embedded rows.

``pair_hash``: a table row chosen by the pair (previous token, token) is added to every embedded row:
row (prev * mul_prev + cur * mul_cur) mod buckets of a table of buckets + 1 rows, whose last row serves a
sequence's first token (it has no predecessor).  The predecessor of a portion's first token is the request's
newest token of an earlier step: one int32 per request slot, kept on the device and renewed by the kernel, so a
token that was sampled on the device and not yet read by the host can be the predecessor too.  The reference
has no such table (its embedding is the lookup alone: crates/thuban_kernel/wgsl/embed.wgsl:15-33).
"""
from __future__ import annotations

import torch

from ..cache.manager import StateSpec
from ..errors import ConfigError
from ..registry import EMBED_ADDITIONS
from .base import EmbedAddition, mat


@EMBED_ADDITIONS.register("pair_hash")
class PairHashEmbedding(EmbedAddition):
    """params: hidden_size, buckets, mul_prev, mul_cur, tensor (name of the table, default "table").
    tensor: [buckets + 1, hidden_size]."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.buckets = int(params["buckets"])
        self.mul_prev, self.mul_cur = int(params["mul_prev"]), int(params["mul_cur"])
        self.tensor = str(params.get("tensor", "table"))
        if self.buckets < 1:
            raise ConfigError(f"pair_hash: buckets must be positive, got {self.buckets}")
        if self.mul_prev < 0 or self.mul_cur < 0:
            raise ConfigError("pair_hash: the multipliers must not be negative")
        self.table = None

    def weights(self):
        return {self.tensor: mat(self.buckets + 1, self.hidden)}

    def load(self, tensors):
        self.table = tensors[self.tensor]

    def state_spec(self):
        return StateSpec((), torch.int32)        # the request's newest token

    def forward(self, h, step, state, fed_from=None):
        fed = fed_from is not None and step.fed_rows is not None
        self.ops.pair_embed_add(step.ids, step.pos, step.slot, state, self.table, h, self.mul_prev, self.mul_cur,
                                fed_rows=step.fed_rows if fed else None, fed_from=fed_from if fed else None)
