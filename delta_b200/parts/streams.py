"""Residual streams, the mixing of several stream copies, and the block that runs on them.

``single``: one copy of the stream in the compute type; a block hands its last update on as ``pending`` and the
next norm adds it (the pre-norm block of ``block.py``).

``mixed_f32``: the stream is kept in 32 bit as S copies X_1..X_S that all start as the embedding output
("hyper-connections"; S = 1 with unit weights is the ordinary residual sum in 32 bit).  A sublayer with the
learned weights r[S], o[S], M[S][S] of its ``StreamMixing`` reads
    u = sum_s r[s] X_s ,        y = sublayer(norm(u)) ,
and then all copies change at once from the old ones,
    X_t <- sum_s M[s][t] X_s + o[t] y .
At the end the copies are summed.  The update of one sublayer and the read of the next are one kernel
(``ops.stream_norm``), so the copies are read and written once per sublayer; ``pending`` is the pair
(y, mixing) whose update has not been applied yet.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import BLOCKS, STREAM_MIXINGS, STREAMS, Block, Part, Stream, TensorSpec
from .norm import RMSNorm


@STREAMS.register("single")
class SingleStream(Stream):
    def __init__(self, width: int):
        self.width = int(width)

    def start(self, ctx, table):
        x = torch.empty((ctx.num_tokens, self.width), dtype=ctx.dtype, device=ctx.device)
        ops.embedding(ctx.tokens, table, x, err=ctx.err)
        return x

    def finish(self, ctx, x, pending, norm, rows):
        return norm.forward(ctx, x, add=pending, rows=rows)

    def total(self, ctx, x, pending):
        return (x.float() + pending.float()) if pending is not None else x.float()


def _update_of(pending):
    if pending is None:
        return None
    y, mixing = pending
    return (y, mixing.mix_w(y.device), mixing.out_w(y.device))


@STREAMS.register("mixed_f32")
class MixedStreams(Stream):
    def __init__(self, width: int, copies: int = 1):
        self.width, self.copies = int(width), int(copies)

    def start(self, ctx, table):
        X = torch.empty((ctx.num_tokens, self.copies, self.width), dtype=torch.float32, device=ctx.device)
        ops.embedding_streams(ctx.tokens, table, X, err=ctx.err)
        return X

    def finish(self, ctx, X, pending, norm, rows):
        if not isinstance(norm, RMSNorm):
            raise TypeError("the mixed stream ends in an RMSNorm")
        out = torch.empty((rows.shape[0], self.width), dtype=ctx.dtype, device=ctx.device)
        return ops.stream_norm(X, out, weight=norm.weight32(), eps=norm.eps, read=None, update=_update_of(pending), rows=rows,
                               write_back=False)

    def total(self, ctx, X, pending):
        out = torch.empty((X.shape[0], self.width), dtype=torch.float32, device=ctx.device)
        return ops.stream_norm(X, out, weight=None, read=None, update=_update_of(pending), write_back=False)


@STREAM_MIXINGS.register("learned")
class StreamMixing(Part):
    """The weights of one sublayer on ``copies`` stream copies: ``<prefix>in`` [S], ``<prefix>out`` [S] and
    ``<prefix>mix`` [S, S] (indexed [from, to]), kept in 32 bit.  ``prefix`` None: unit weights (the plain sum)."""

    def __init__(self, copies: int = 1, prefix: Optional[str] = None):
        self.copies = int(copies)
        self.prefix = prefix
        if prefix is None and self.copies != 1:
            raise ValueError("several stream copies need learned mixing weights")
        self._in = self._out = self._mix = None

    def tensor_specs(self):
        if self.prefix is None:
            return []
        S = self.copies
        return [TensorSpec(self.prefix + "in", (S,), kind="vector", init="uniform:0.2:0.5"),
                TensorSpec(self.prefix + "out", (S,), kind="vector", init="uniform:0.5:1.0"),
                TensorSpec(self.prefix + "mix", (S, S), kind="vector", init="eye:0.1")]

    def bind(self, tensors):
        if self.prefix is not None:
            self._in = tensors[self.prefix + "in"].float().contiguous()
            self._out = tensors[self.prefix + "out"].float().contiguous()
            self._mix = tensors[self.prefix + "mix"].float().contiguous()

    def _unit(self, device):
        if self._in is None or self._in.device != device:
            self._in = torch.ones(1, dtype=torch.float32, device=device)
            self._out = torch.ones(1, dtype=torch.float32, device=device)
            self._mix = torch.ones((1, 1), dtype=torch.float32, device=device)

    def in_w(self, device):
        if self.prefix is None:
            self._unit(device)
        return self._in

    def out_w(self, device):
        if self.prefix is None:
            self._unit(device)
        return self._out

    def mix_w(self, device):
        if self.prefix is None:
            self._unit(device)
        return self._mix

    def read(self, ctx, X, pending, norm):
        """Applies the pending update to the copies and returns norm(sum_s in[s] X_s) in the compute type."""
        if not isinstance(norm, RMSNorm):
            raise TypeError("the mixed stream is read through an RMSNorm")
        out = torch.empty((X.shape[0], X.shape[2]), dtype=ctx.dtype, device=X.device)
        return ops.stream_norm(X, out, weight=norm.weight32(), eps=norm.eps, read=self.in_w(X.device), update=_update_of(pending))


@BLOCKS.register("stream_pre_norm")
class StreamPreNormBlock(Block):
    """Pre-norm sublayers on a mixed stream: the mixer, and a feed-forward when the layer has one."""
    roles = ("norm1", "mixer", "mixing1")
    optional_roles = ("norm2", "feed_forward", "mixing2")

    def __init__(self, parts):
        super().__init__(parts)
        if (self.feed_forward is None) != (self.norm2 is None) or (self.feed_forward is None) != (self.mixing2 is None):
            raise ValueError("a feed-forward sublayer needs norm2, feed_forward and mixing2 together")

    def forward(self, ctx, X, pending, cache):
        a = self.mixing1.read(ctx, X, pending, self.norm1)
        pending = (self.mixer.forward(ctx, a, cache), self.mixing1)
        if self.feed_forward is not None:
            f = self.mixing2.read(ctx, X, pending, self.norm2)
            pending = (self.feed_forward.forward(ctx, f), self.mixing2)
        return X, pending
