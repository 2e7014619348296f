"""A residual stream of one copy kept in 32 bit, and the block whose sublayers run side by side on it.

``residual_f32``: x [T, d] float32.  It starts as
    x = table[token] * scale  (+ pair_table[(previous token * mul_prev + token * mul_cur) mod buckets])
where the pair table ("bigram embedding") is optional; a request's first token takes the table's last row, and the
token before a portion's first one is per-request state (``stream.prev_token``).  What a layer hands on as ``pending`` is
a ``Pending``: the outputs of its sublayers, not yet added, and what a re-entry adds.  The next norm adds them while it
reads the stream (one kernel, ``ops.residual_norm``): x <- x + (y1 + y2), then + the embedding output, then + the pass's
vector.  ``reentry`` describes a span of layers that runs several times: before every pass but the first the embedding
output (x as ``start`` made it) is added, and before every pass t the row t of the tensor ``reentry["name"]``
[passes, d].

``parallel`` block: h = norm1(x); x <- x + (mixer(h) + feed_forward(h)); one norm, both sublayers read it; the
feed-forward may be absent.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..kernels import ops
from .base import BLOCKS, STREAMS, Block, StateSpec, Stream, TensorSpec

PREV_TOKEN = "stream.prev_token"
KEPT = "residual.embedding_output"


@dataclass
class Pending:
    """What has not been added to the stream yet."""
    updates: tuple = ()                       # outputs of the last layer's sublayers [T, d], compute type
    extra: Optional[torch.Tensor] = None      # float32 [T, d]
    vec: Optional[torch.Tensor] = None        # float32 [d]

    def empty(self) -> bool:
        return not self.updates and self.extra is None and self.vec is None


def read(ctx, x, pending: Optional[Pending], norm, rows=None, write_back=True):
    """Settles ``pending`` into x and returns norm(x) in the compute type (``norm``: a part with ``weight32()``, ``eps`` and
    ``kind``; None: the settled x itself in float32)."""
    p = pending or Pending()
    n = x.shape[0] if rows is None else rows.shape[0]
    if norm is None:
        out = torch.empty((n, x.shape[1]), dtype=torch.float32, device=x.device)
        return ops.residual_norm(x, out, updates=p.updates, extra=p.extra, vec=p.vec, rows=rows, write_back=write_back)
    out = torch.empty((n, x.shape[1]), dtype=ctx.dtype, device=x.device)
    return ops.residual_norm(x, out, updates=p.updates, extra=p.extra, vec=p.vec, weight=norm.weight32(), eps=norm.eps, kind=norm.kind,
                             rows=rows, write_back=write_back)


@STREAMS.register("residual_f32")
class ResidualStream(Stream):
    def __init__(self, width: int, scale: float = 1.0, pair: Optional[dict] = None, reentry: Optional[dict] = None):
        """``pair``: {name, buckets, mul_prev, mul_cur} of the hashed pair table [buckets + 1, d] (None: none).
        ``reentry``: {name, passes, add_embedding} (None: no span runs more than once)."""
        self.width, self.scale = int(width), float(scale)
        self.pair = dict(pair) if pair else None
        self.reentry = dict(reentry) if reentry else None
        self.pair_table = self.pass_vectors = None

    def tensor_specs(self):
        specs = []
        if self.pair:
            specs.append(TensorSpec(self.pair["name"], (int(self.pair["buckets"]) + 1, self.width), kind="table"))
        if self.reentry:
            specs.append(TensorSpec(self.reentry["name"], (int(self.reentry["passes"]), self.width), kind="vector", init="normal"))
        return specs

    def bind(self, tensors):
        if self.pair:
            self.pair_table = tensors[self.pair["name"]]
        if self.reentry:
            self.pass_vectors = tensors[self.reentry["name"]].float().contiguous()

    def state_specs(self):
        return {PREV_TOKEN: StateSpec((1,), torch.int32, -1)} if self.pair else {}

    def _keeps(self) -> bool:
        return bool(self.reentry and self.reentry.get("add_embedding", True) and int(self.reentry["passes"]) > 1)

    def start(self, ctx, table):
        T = ctx.num_tokens
        x = torch.empty((T, self.width), dtype=torch.float32, device=ctx.device)
        keep = None
        if self._keeps():
            keep = ctx.scratch(KEPT, (T, self.width), torch.float32, bound=(ctx.max_step_tokens, self.width))
        pair = self.pair or {}
        state = ctx.state(PREV_TOKEN) if self.pair else None
        ops.embedding_pair(ctx.tokens, table, x, scale=self.scale, pair_table=self.pair_table, buckets=pair.get("buckets", 0),
                           mul_prev=pair.get("mul_prev", 0), mul_cur=pair.get("mul_cur", 0), prev_state=state, tok_row=ctx.tok_row,
                           tok_pos=ctx.tok_pos, row_q_start=ctx.row_q_start, row_slot=ctx.row_slot, keep=keep, err=ctx.err)
        if self.pair:
            ops.remember_tokens(ctx.tokens, state, row_q_start=ctx.row_q_start, row_q_len=ctx.row_q_len, row_slot=ctx.row_slot)
        self._kept = keep
        return x

    def enter_pass(self, ctx, x, pending, number: int):
        if not self.reentry:
            raise ValueError("the stream was built without a re-entry and is told that a pass starts")
        p = pending or Pending()
        if p.extra is not None or p.vec is not None:      # two re-entries without a layer between them: settle the first
            ops.residual_norm(x, None, updates=p.updates, extra=p.extra, vec=p.vec)
            p = Pending()
        extra = self._kept if (number > 0 and self._keeps()) else None
        return x, Pending(p.updates, extra, self.pass_vectors[number])

    def finish(self, ctx, x, pending, norm, rows):
        return read(ctx, x, pending, norm, rows=rows, write_back=False)

    def total(self, ctx, x, pending):
        return read(ctx, x, pending, None, write_back=False)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    """One norm whose output the mixer and the feed-forward both read; their outputs are summed into the stream."""
    roles = ("norm1", "mixer")
    optional_roles = ("feed_forward",)

    def forward(self, ctx, x, pending, cache):
        h = read(ctx, x, pending, self.norm1)
        ys = (self.mixer.forward(ctx, h, cache),)
        if self.feed_forward is not None:
            ys = ys + (self.feed_forward.forward(ctx, h),)
        return x, Pending(ys)
