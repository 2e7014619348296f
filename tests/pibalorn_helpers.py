"""Small Pibalorn configurations and weights for the tests.  Tensor names and shapes are written out here from the
configuration, independently of the engine's own list, so a name or shape the engine gets wrong shows as a loading
error."""
from __future__ import annotations

import math

import torch

from roletar_helpers import write_folder  # noqa: F401  (the folder writer knows no design)


def attention(heads, kv_heads, dim, scale=None, rot_dims=None, base=10000.0):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale if scale is not None else 1.0 / math.sqrt(dim))
    if rot_dims:
        m["rot"] = dict(base=base, dims=rot_dims)
    return dict(type="attention", mixer=m)


def lightning(heads, dim, vdim, decay):
    return dict(type="lightning", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay)))


def dense(layer, ff, limit):
    return dict(layer, mlp=dict(kind="dense", ff=ff, limit=limit))


def moe(layer, experts, top, ff, limit, shared=None):
    mlp = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff, limit=limit) if limit is not None else dict(ff=ff))
    if shared:
        mlp["shared"] = dict(ff=shared[0], limit=shared[1])
    return dict(layer, mlp=mlp)


def bare(layer):
    return dict(layer, mlp=None)


def config(which: str) -> dict:
    base = dict(architecture="Pibalorn", norm=dict(eps=1e-5))
    if which == "mix":      # both mixers, both feed-forwards, a layer without one, a loop in the middle, a pair table
        return dict(base, vocab=300, width=96, embedding=dict(scale=3.0, bigram=dict(buckets=211, mul_prev=31, mul_cur=7)),
                    loop=dict(start=1, stop=3, times=2), layers=[
            dense(lightning(3, 16, 24, (0.5, 0.9, 0.995)), 80, 1.2),
            moe(attention(4, 2, 24, 0.2, rot_dims=16, base=1000.0), 6, 2, 40, 0.9, shared=(56, 1.4)),
            moe(lightning(2, 24, 16, (0.97, 0.7)), 5, 3, 24, 1.1),
            bare(attention(2, 2, 16, 0.3, rot_dims=16))])
    if which == "odd":      # no size a multiple of 4; the loop starts at layer 0 and runs three times; every expert is chosen
        return dict(base, vocab=61, width=50, norm=dict(eps=1e-6), embedding=dict(scale=1.7, bigram=dict(buckets=13, mul_prev=5, mul_cur=3)),
                    loop=dict(start=0, stop=2, times=3), layers=[
            moe(attention(3, 1, 10, 0.35, rot_dims=6, base=300.0), 5, 5, 9, 0.8, shared=(14, 2.0)),
            dense(lightning(3, 6, 10, (0.8, 0.99, 0.3)), 30, 1.0),
            dense(attention(2, 2, 6, 0.5, rot_dims=2, base=50.0), 18, 0.7)])
    if which == "one":      # what other models make larger is 1 or absent here: one head, one expert chosen, one pass, no pair
        return dict(base, vocab=128, width=48, loop=dict(start=1, stop=2, times=1), layers=[    # table, no embedding key, no rotation
            moe(attention(1, 1, 8, 0.6), 3, 1, 16, 1.5),
            bare(lightning(1, 8, 8, (0.9,))),
            moe(attention(4, 4, 12, 0.25, rot_dims=8), 1, 1, 20, 1.0, shared=(8, 1.0))])
    if which == "sharp":    # a large scale on unit-normed heads: single far keys carry most of the weight; tiny pages
        return dict(base, vocab=97, width=64, embedding=dict(scale=2.0), layers=[
            bare(attention(4, 2, 16, 1.5, rot_dims=8, base=100.0)), bare(attention(2, 1, 32, 1.0, rot_dims=32, base=20000.0))])
    if which == "wide":     # sizes that the tensor-core kernels take (multiples of 64): long portions send the experts' products to the
        return dict(base, vocab=200, width=128, embedding=dict(scale=2.0), layers=[      # tcgen05 kernel, short ones to warp-level MMA
            moe(lightning(2, 64, 64, (0.98, 0.8)), 4, 2, 64, 1.1, shared=(64, 1.3)),
            moe(attention(4, 2, 32, 0.3, rot_dims=16, base=5000.0), 3, 1, 128, 0.9)])
    if which == "only_attention":
        return dict(base, vocab=97, width=40, layers=[bare(attention(4, 2, 16, 0.4, rot_dims=12, base=500.0))])
    if which == "only_lightning":
        return dict(base, vocab=97, width=40, layers=[bare(lightning(2, 16, 8, (0.95, 0.6)))])
    if which == "only_experts":   # the mixer is tiny, the experts dominate
        return dict(base, vocab=97, width=40, layers=[moe(lightning(1, 4, 4, (0.5,)), 7, 3, 24, 1.0, shared=(16, 1.5)),
                                                     moe(lightning(1, 4, 4, (0.5,)), 4, 2, 12, None)])   # (no limit given: nothing is clamped)
    if which == "only_pairs":     # the pair table and the re-entries dominate: one small layer run four times
        return dict(base, vocab=97, width=40, embedding=dict(scale=0.5, bigram=dict(buckets=1, mul_prev=1, mul_cur=1)),
                    loop=dict(start=0, stop=1, times=4), layers=[dense(attention(1, 1, 8, 0.3, rot_dims=4), 24, 1.0)])
    if which == "pairs_many":     # more buckets than (previous, current) products can overflow 32 bits with
        return dict(base, vocab=250, width=32, embedding=dict(scale=1.0, bigram=dict(buckets=9973, mul_prev=100003, mul_cur=99991)),
                    layers=[bare(lightning(2, 8, 8, (0.9, 0.8)))])
    raise KeyError(which)


PAGE_SIZE = {"wide": 16, "mix": 16, "odd": 2, "one": 4, "sharp": 4, "only_attention": 8, "only_lightning": 16, "only_experts": 16, "only_pairs": 8,
             "pairs_many": 16}


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> float32 tensor whose values are all representable in bfloat16."""
    g = torch.Generator().manual_seed(seed)
    d = cfg["width"]

    def mat(out, inp, gain=1.0):
        return torch.randn(out, inp, generator=g) * (gain / math.sqrt(inp))

    def uni(shape, a, b):
        return a + (b - a) * torch.rand(shape, generator=g)

    W = {"embed": torch.randn(cfg["vocab"], d, generator=g), "head": mat(cfg["vocab"], d, 2.0), "final.norm": uni((d,), 0.8, 1.2)}
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        W["bigram"] = torch.randn(bg["buckets"] + 1, d, generator=g) * 1.5
    if cfg.get("loop"):
        W["loop.step"] = torch.randn(cfg["loop"]["times"], d, generator=g)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"] = uni((d,), 0.8, 1.2)
        if L["type"] == "attention":
            H, G, dk = m["heads"], m["kv_heads"], m["dim"]
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.o"] = mat(H * dk, d, 2.0), mat(G * dk, d, 2.0), mat(d, H * dk)
        else:
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            W[p + "mix.q"], W[p + "mix.k"] = mat(H * dk, d, 1.5), mat(H * dk, d, 1.5)
            W[p + "mix.v"], W[p + "mix.g"] = mat(H * dv, d, 1.5), mat(H * dv, d, 2.0)
            W[p + "mix.norm"], W[p + "mix.o"] = uni((H * dv,), 0.8, 1.2), mat(d, H * dv)
        mlp = L.get("mlp")
        if not mlp:
            continue

        def glu(q, ff):
            W[q + "gate"], W[q + "up"], W[q + "down"] = mat(ff, d, 2.0), mat(ff, d, 2.0), mat(d, ff)

        if mlp["kind"] == "dense":
            glu(p + "mlp.", mlp["ff"])
        else:
            W[p + "mlp.router"] = mat(mlp["router"]["experts"], d, 3.0)
            for e in range(mlp["router"]["experts"]):
                glu(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
            if mlp.get("shared"):
                glu(p + "mlp.shared.", mlp["shared"]["ff"])
                W[p + "mlp.shared.sg"] = mat(1, d, 2.0)
    return {k: v.to(torch.bfloat16).float() for k, v in W.items()}
