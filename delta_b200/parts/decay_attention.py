"""Linear attention with a constant decay per head ("lightning attention").

With mixer input h, H heads, key size dk and value size dv:
    q = act(W_q h), k = act(W_k h)  [H, dk],   v = act(W_v h)  [H, dv]        act = silu
    S_h <- decay_h * S_h + k_h v_h^T ,   o_h = S_h^T q_h                       per head, token by token
    out = W_o ( rmsnorm(o over all heads) * w * sigmoid(W_g h) )
A request's state is S [H, dk, dv] in 32 bit, zero at its start, one per run of the layer; a step continues from what
the request's earlier steps left, so a prompt may be cut anywhere.  The four projections are one product; the
recurrence, its decays and the norm are 32 bit whatever the compute type.  Steps of single tokens stream the state through
registers once; short portions run one block per (row, head) over the row's chunks in turn; long portions run their chunks in parallel (``csrc/decay_attention.cu``).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from . import linear
from .base import MIXERS, Mixer, StateSpec, TensorSpec

STATE = "decay_attention"
PARALLEL_FROM = 65      # portions of at least this many tokens run their chunks in parallel


@MIXERS.register("decay_attention")
class DecayAttention(Mixer):
    """Tensor names under ``prefix``: ``q``, ``k`` [H*dk, d], ``v``, ``g`` [H*dv, d], ``norm`` [H*dv], ``o`` [d, H*dv]."""

    def __init__(self, prefix: str, width: int, heads: int, head_dim: int, value_dim: int, decays, eps: float):
        self.prefix, self.width = prefix, int(width)
        self.heads, self.dk, self.dv = int(heads), int(head_dim), int(value_dim)
        self.decays = [float(x) for x in decays]
        if len(self.decays) != self.heads:
            raise ValueError(f"{len(self.decays)} decays for {self.heads} heads")
        self.eps = float(eps)
        self.w_in = self.w_o = self.norm_w = self._decays = None

    def tensor_specs(self):
        p, d, H, dk, dv = self.prefix, self.width, self.heads, self.dk, self.dv
        return [TensorSpec(p + "q", (H * dk, d)), TensorSpec(p + "k", (H * dk, d)), TensorSpec(p + "v", (H * dv, d)),
                TensorSpec(p + "g", (H * dv, d)), TensorSpec(p + "norm", (H * dv,), kind="vector", init="norm"),
                TensorSpec(p + "o", (d, H * dv))]

    def bind(self, tensors):
        p = self.prefix
        self.w_in = torch.cat([tensors[p + "q"], tensors[p + "k"], tensors[p + "v"], tensors[p + "g"]], dim=0).contiguous()
        self.w_o = tensors[p + "o"]
        self.norm_w = tensors[p + "norm"].float().contiguous()
        self._decays = torch.tensor(self.decays, dtype=torch.float64, device=self.w_o.device)

    def run_state_specs(self):
        return {STATE: StateSpec((self.heads, self.dk, self.dv), torch.float32, 0.0)}

    def forward(self, ctx, x, cache):
        H, dk, dv = self.heads, self.dk, self.dv
        T = x.shape[0]
        qkvg = linear.linear(ctx, x, self.w_in)                       # [T, 2 H dk + 2 H dv]: q | k | v | g, before activations
        o = torch.empty((T, H * dv), dtype=torch.float32, device=x.device)
        rows = dict(row_slot=ctx.row_slot, row_q_start=ctx.row_q_start, row_q_len=ctx.row_q_len)
        if not ctx.replayable and ctx.max_q_len >= PARALLEL_FROM and ops.decay_attention_chunked_supported(dk, dv):
            # long portions: the recurrence is linear in the state, so a row's chunks run in parallel and are stitched together
            chunk = ops.decay_attention_chunk()

            def layout():
                counts = [-(-n // chunk) for n in ctx.host["q_lens"]]
                base = [sum(counts[:i]) for i in range(len(counts))]
                return torch.tensor(base, dtype=torch.int32).to(x.device, non_blocking=True), sum(counts), max(counts)
            base, total, most = ctx.memo(("decay_attention chunks", chunk), layout)
            bound = (-(-ctx.max_step_tokens // chunk) + ctx.max_rows) * H * dk * dv
            work = ctx.scratch("decay_attention.chunks", (total * H * dk * dv,), torch.float32, bound=(bound,))
            ops.decay_attention_chunked(qkvg, 0, H * dk, 2 * H * dk, self._decays, cache.state[STATE], o, work, base, most, H=H, dk=dk,
                                        dv=dv, silu=True, **rows)
        elif ctx.decode_only and ops.decay_attention_step_supported(dk, dv):
            ops.decay_attention_step(qkvg, 0, H * dk, 2 * H * dk, self._decays, cache.state[STATE], o, H=H, dk=dk, dv=dv, silu=True,
                                     row_slot=ctx.row_slot, row_q_start=ctx.row_q_start)
        else:
            ops.decay_attention(qkvg, 0, H * dk, 2 * H * dk, self._decays, cache.state[STATE], o, H=H, dk=dk, dv=dv, silu=True, **rows)
        y = torch.empty((T, H * dv), dtype=x.dtype, device=x.device)
        g_at = qkvg.data_ptr() + (2 * H * dk + H * dv) * qkvg.element_size()
        ops.gated_rms_norm(o, g_at, qkvg.shape[1], self.norm_w, y, self.eps)
        return linear.linear(ctx, y, self.w_o)
