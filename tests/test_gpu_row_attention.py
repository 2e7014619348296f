"""The attention kernels over a cache of rows against the softmax written out in float64: key and value of
different sizes, a value that is the front part of its key (the latent cache), windows, sinks, shuffled pages,
prompt portions beside single tokens.  Queries and keys are made so that one key's score stands out: a key that
a kernel misses (far back, at a page border, at the window's edge) or wrongly sees changes the whole output."""
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


class Ctx:
    """The little of a step's context that the kernel choice reads."""
    def __init__(self, q_lens, dtype, plain):
        self.dtype = DT[dtype]
        self.plain_kernels = {"attention"} if plain else set()
        self.decode_only = all(n == 1 for n in q_lens)
        self.host = dict(q_lens=q_lens)
        self.max_q_len = max(q_lens)
        self.max_seq_len = 0
        self.sm_count = torch.cuda.get_device_properties(0).multi_processor_count
        self._scratch = {}

    def scratch(self, key, shape, dtype, bound=None):
        n = 1
        for s in shape:
            n *= int(s)
        if key not in self._scratch or self._scratch[key].numel() < n:
            self._scratch[key] = torch.empty(max(n, 1), dtype=dtype, device="cuda")
        return self._scratch[key][:n].view(*shape)


def reference(rows, H, KV, dk, dv, scale, window, sink, latent):
    out = []
    for (before, n, Q, K, V) in rows:
        Q, K, V = Q.double(), K.double(), V.double()
        o = torch.zeros(n, H, dv, dtype=torch.float64)
        for i in range(n):
            pos = before + i
            lo = max(0, pos - window + 1) if window else 0
            for h in range(H):
                g = h // (H // KV)
                s = (K[lo:pos + 1, g] @ Q[i, h]) * scale
                m = s.max() if sink is None else torch.maximum(s.max(), sink[h].double())
                e = torch.exp(s - m)
                den = e.sum() + (torch.exp(sink[h].double() - m) if sink is not None else 0.0)
                o[i, h] = (e / den) @ V[lo:pos + 1, g]
        out.append(o)
    return torch.cat(out)


def run_case(dtype, plain, shape, row_lens, window=None, use_sink=False, latent=False, spikes=(), seed=0, ps=16):
    """``row_lens``: (tokens cached before the step, new tokens) per batch row.  ``spikes``: (row, query index, key
    position): that query and that key get a large common component."""
    from delta_b200.kernels import ops
    from delta_b200.parts import row_attention
    H, KV, dk, dv = shape
    dt = DT[dtype]
    g = torch.Generator().manual_seed(seed)
    rows = []
    for r, (before, n) in enumerate(row_lens):
        L = before + n
        Q = torch.randn(n, H, dk, generator=g)
        K = torch.randn(L, KV, dk, generator=g)
        V = torch.randn(L, KV, dk if latent else dv, generator=g)
        for (rr, qi, kp) in spikes:
            if rr == r:
                K[kp, :, 0] += 12.0
                Q[qi, :, 0] += 12.0
        Q, K, V = (t.to(dt).float() for t in (Q, K, V))
        if latent:
            V = K[..., :dv].clone()
        rows.append((before, n, Q, K, V))
    scale = 1.0 / math.sqrt(dk)
    sink = (torch.randn(H, generator=g) * 1.5) if use_sink else None
    want = reference(rows, H, KV, dk, dv, scale, window, sink, latent)
    # the cache, pages handed out in a shuffled order
    row_width = dk if latent else dk + dv
    k_off, v_off = 0, (0 if latent else dk)
    n_pages = sum((b + n + ps - 1) // ps for b, n in row_lens) + 3
    order = list(range(n_pages))
    random.Random(seed).shuffle(order)
    cache = torch.zeros(n_pages, KV, ps, row_width, dtype=dt)
    max_pages = max((b + n + ps - 1) // ps for b, n in row_lens)
    bt = torch.full((len(row_lens), max_pages), -1, dtype=torch.int32)
    nxt = 0
    for r, (before, n, Q, K, V) in enumerate(rows):
        for lp in range((before + n + ps - 1) // ps):
            bt[r, lp] = order[nxt]
            nxt += 1
        for j in range(before + n):
            page, off = int(bt[r, j // ps]), j % ps
            cache[page, :, off, k_off:k_off + dk] = K[j].to(dt)
            if not latent:
                cache[page, :, off, v_off:v_off + dv] = V[j].to(dt)
    q = torch.cat([Q.reshape(n, H * dk) for (_, n, Q, _, _) in rows]).to(dt).cuda()
    q_lens = [n for _, n in row_lens]
    starts = [sum(q_lens[:i]) for i in range(len(q_lens))]
    i32 = dict(dtype=torch.int32, device="cuda")
    tok_row = torch.tensor([r for r, n in enumerate(q_lens) for _ in range(n)], **i32)
    tok_pos = torch.tensor([b + i for (b, n) in row_lens for i in range(n)], **i32)
    out = torch.zeros(sum(q_lens), H * dv, dtype=dt, device="cuda")
    err = ops.new_error_record("cuda")
    ctx = Ctx(q_lens, dtype, plain)
    ctx.max_seq_len = max(b + n for b, n in row_lens)
    # (the parameters hold raw addresses: every device tensor stays referenced until the result is read)
    dev = dict(cache=cache.cuda(), block_table=bt.cuda(), row_q_start=torch.tensor(starts, **i32), row_q_len=torch.tensor(q_lens, **i32),
               row_pos_start=torch.tensor([b for b, _ in row_lens], **i32), sink=sink.cuda() if sink is not None else None)
    params = ops.row_attn_params(q=q, q_stride=H * dk, q_head_stride=dk, out=out, tok_row=tok_row, tok_pos=tok_pos, H=H, KV=KV, dk=dk,
                                 dv=dv, ps=ps, row_width=row_width, k_off=k_off, v_off=v_off, scale=scale, window=window or 0, err=err,
                                 **dev)
    ctx.err = err
    row_attention.run(ctx, params)
    ops.raise_if_error(err)
    got = out.float().cpu().view(-1, H, dv).double()
    del dev
    worst = (got - want).abs().max().item()
    assert worst <= TOL[dtype] * max(1.0, want.abs().max().item()), f"differs by {worst:.3e}"
    return worst


KERNELS = [("float32", True), ("bfloat16", True), ("bfloat16", False)]     # (precision, the plain kernel)


@pytest.mark.parametrize("dtype,plain", KERNELS)
@pytest.mark.parametrize("shape", [(6, 2, 64, 32), (4, 4, 32, 48), (3, 1, 16, 16), (8, 2, 128, 128)])
def test_prompts_and_single_tokens(dtype, plain, shape):
    run_case(dtype, plain, shape, [(0, 70), (33, 1), (0, 2), (100, 37), (15, 1)], seed=1)
    run_case(dtype, plain, shape, [(130, 1), (0, 1), (17, 1)], use_sink=True, seed=2)
    run_case(dtype, plain, shape, [(0, 150)], use_sink=True, window=40, seed=3, ps=8)


@pytest.mark.parametrize("dtype,plain", KERNELS)
@pytest.mark.parametrize("shape", [(4, 1, 80, 64), (16, 1, 160, 128), (2, 1, 48, 32)])
def test_value_is_the_front_of_the_key(dtype, plain, shape):
    run_case(dtype, plain, shape, [(0, 45), (70, 1), (9, 20)], latent=True, seed=4)
    run_case(dtype, plain, shape, [(200, 1), (31, 1)], latent=True, seed=5)


@pytest.mark.parametrize("dtype,plain", KERNELS)
def test_one_key_that_matters(dtype, plain):
    shape, W, ps = (6, 2, 64, 32), 40, 16
    # in a prompt portion: a far key, keys at both sides of page borders, the first tokens
    for kp in (0, 1, ps - 1, ps, 3 * ps - 1, 3 * ps, 200, 298):
        run_case(dtype, plain, shape, [(150, 150)], spikes=[(0, 149, kp)], seed=kp)
    # decoded alone: the same, among hundreds of keys
    for kp in (0, ps - 1, ps, 255, 256, 400, 519):
        run_case(dtype, plain, shape, [(520, 1), (3, 1)], spikes=[(0, 0, kp)], use_sink=True, seed=kp)
    # the window's edge: the last key inside, the first outside, in a portion and decoded alone
    for inside in (True, False):
        for before, n, qi in ((60, 50, 49), (109, 1, 0), (0, 90, 89), (W - 1, 1, 0), (W, 1, 0)):
            pos = before + qi
            kp = pos - W + 1 if inside else pos - W
            if kp < 0:
                continue
            run_case(dtype, plain, shape, [(before, n), (5, 3)], window=W, use_sink=True, spikes=[(0, qi, kp)], seed=pos)
