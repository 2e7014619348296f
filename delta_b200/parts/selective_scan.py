"""The selective state-space mixer (Mamba-1 kind).

With mixer input h, C = ``inner`` channels, N = ``state`` states per channel, a convolution of ``conv`` taps:
    [x | z]      = W_in h
    x            = silu(causal_conv(x) + b)                  per channel over the request's tokens
    [dt | B | C] = W_x x                                     dt_rank + N + N entries
    dt           = softplus(W_dt dt + b_dt)                  one step size per channel
    S[c, n]     <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n ,  A = -exp(A_log)
    y_c          = sum_n S[c, n] C_n + D_c x_c
    out          = W_o (y * silu(z))
A request's state is the last ``conv - 1`` inputs of the convolution and S, both in 32 bit and one pair per run
of the layer; a step continues from what the request's earlier steps left, so a prompt may be cut anywhere.
Step sizes, decays and the state are 32 bit; the products run in the compute type.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from . import linear
from .base import MIXERS, Mixer, StateSpec, TensorSpec

SEGMENT = 128           # tokens of a segment when a long portion's recurrence is run in parallel pieces
CONV_STATE = "conv"
SCAN_STATE = "scan"


@MIXERS.register("selective_scan")
class SelectiveScan(Mixer):
    """Tensor names under ``prefix``: ``in`` [2C, d], ``conv`` [C, taps], ``conv.b`` [C], ``x`` [dt_rank + 2N, C],
    ``dt`` [C, dt_rank], ``dt.b`` [C], ``A_log`` [C, N], ``D`` [C], ``o`` [d, C]."""

    def __init__(self, prefix: str, width: int, inner: int, state: int, conv: int, dt_rank: int):
        self.prefix, self.width = prefix, int(width)
        self.inner, self.state, self.taps, self.dt_rank = int(inner), int(state), int(conv), int(dt_rank)
        if self.taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.w_in = self.w_x = self.w_dt = self.w_o = None
        self.conv_w = self.conv_b = self.dt_b = self.A_log = self.D = None

    def tensor_specs(self):
        p, d, C, N, r = self.prefix, self.width, self.inner, self.state, self.dt_rank
        return [TensorSpec(p + "in", (2 * C, d)), TensorSpec(p + "conv", (C, self.taps), kind="vector", init="uniform:-0.5:0.5"),
                TensorSpec(p + "conv.b", (C,), kind="vector", init="uniform:-0.1:0.1"), TensorSpec(p + "x", (r + 2 * N, C)),
                TensorSpec(p + "dt", (C, r)), TensorSpec(p + "dt.b", (C,), kind="vector", init="uniform:-4:-1"),
                TensorSpec(p + "A_log", (C, N), kind="vector", init="uniform:-1:1.5"),
                TensorSpec(p + "D", (C,), kind="vector", init="norm"), TensorSpec(p + "o", (d, C))]

    def bind(self, tensors):
        p = self.prefix
        self.w_in, self.w_x, self.w_dt, self.w_o = tensors[p + "in"], tensors[p + "x"], tensors[p + "dt"], tensors[p + "o"]
        f = lambda n: tensors[p + n].float().contiguous()   # noqa: E731  (what the recurrence reads is kept in 32 bit)
        self.conv_w, self.conv_b, self.dt_b, self.A_log, self.D = f("conv"), f("conv.b"), f("dt.b"), f("A_log"), f("D")

    def run_state_specs(self):
        return {CONV_STATE: StateSpec((max(self.taps - 1, 1), self.inner), torch.float32, 0.0),
                SCAN_STATE: StateSpec((self.inner, self.state), torch.float32, 0.0)}

    def forward(self, ctx, x, cache):
        C, N, r = self.inner, self.state, self.dt_rank
        T = x.shape[0]
        rows = dict(row_slot=ctx.row_slot, row_q_start=ctx.row_q_start, row_q_len=ctx.row_q_len)
        xz = linear.linear(ctx, x, self.w_in)                                   # [T, 2C]: x | z
        xc = torch.empty((T, C), dtype=x.dtype, device=x.device)
        ops.conv_silu(xz, 2 * C, self.conv_w, self.conv_b, cache.state[CONV_STATE], xc, tok_row=ctx.tok_row, **rows)
        low = linear.linear(ctx, xc, self.w_x)                                  # [T, r + 2N]: dt | B | C
        dtraw = linear.linear(ctx, low[:, :r].contiguous(), self.w_dt)          # [T, C], before the bias and softplus
        y = torch.empty((T, C), dtype=x.dtype, device=x.device)
        seg = {}
        if not ctx.replayable and ctx.max_q_len > SEGMENT:
            # long portions: the recurrence is linear, so segments of a row run in parallel and are stitched together
            segs = -(-ctx.max_q_len // SEGMENT)
            n = ctx.num_rows * segs
            seg = dict(seg_len=SEGMENT, segs=segs, seg_state=ctx.scratch("selective_scan.segments", (n, C, N), torch.float32),
                       seg_dt=ctx.scratch("selective_scan.segment_dt", (n, C), torch.float32))
        ops.selective_scan(xc, dtraw, low, r, r + N, xz.data_ptr() + C * xz.element_size(), 2 * C, self.A_log, self.D, self.dt_b,
                           cache.state[SCAN_STATE], y, **rows, **seg)
        return linear.linear(ctx, y, self.w_o)
