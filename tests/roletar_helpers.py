"""Small Roletar configurations and weights for the tests.  Tensor names and shapes are written out here from
the configuration, independently of the engine's own list, so a name or shape the engine gets wrong shows as a
loading error."""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def attention(heads, kv_heads, dim, vdim, window, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale if scale is not None else 1.0 / math.sqrt(dim))
    if window is not None:
        m["mask"] = dict(size=window)
    return dict(type="attention", mixer=m)


def latent(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, dims=None, scale=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank,
             scale=scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim), rot=dict(base=base, dims=dims or rot_dim))
    return dict(type="latent_attention", mixer=m)


def mamba(inner, state, conv, dt_rank):
    return dict(type="mamba1", mixer=dict(inner=inner, state=state, conv=conv, dt_rank=dt_rank))


def with_mlp(layer, ff):
    return dict(layer, mlp=dict(kind="dense", ff=ff) if ff else None)


def config(which: str) -> dict:
    base = dict(architecture="Roletar", norm=dict(eps=1e-5))
    if which == "mix":      # every mixer, a loop over the recurrent and the windowed layer, three streams, a soft cap
        return dict(base, vocab=300, width=96, streams=3, logit_softcap=20.0, loop=dict(start=0, stop=2, times=2), layers=[
            with_mlp(mamba(160, 12, 3, 6), 200), with_mlp(attention(4, 2, 24, 40, 21, 0.3), None),
            with_mlp(latent(3, 16, 8, 24, 40, base=1000.0, scale=0.25), 128)])
    if which == "plain":    # no streams key, no loop, no cap; partial rotation; a window longer than any prompt; one tap
        return dict(base, vocab=211, width=64, norm=dict(eps=1e-6), layers=[
            with_mlp(latent(2, 24, 16, 16, 24, base=50.0, dims=8), 96), with_mlp(attention(3, 3, 16, 16, 4096), 80),
            with_mlp(mamba(72, 40, 1, 1), None), with_mlp(attention(2, 1, 32, 8, None), None)])
    if which == "one":      # one learned stream copy, a loop of one layer run three times, many states, one head
        return dict(base, vocab=128, width=48, streams=1, logit_softcap=5.0, loop=dict(start=1, stop=2, times=3), layers=[
            with_mlp(attention(1, 1, 8, 24, 9, 0.5), 64), with_mlp(mamba(56, 70, 5, 3), 64),
            with_mlp(latent(1, 8, 4, 8, 12, base=10000.0), None)])
    if which == "only_mamba":
        return dict(base, vocab=97, width=40, streams=2, layers=[with_mlp(mamba(64, 16, 4, 4), None)])
    if which == "only_attention":
        return dict(base, vocab=97, width=40, streams=2, layers=[with_mlp(attention(4, 2, 16, 8, 13, 0.4), None)])
    if which == "only_latent":
        return dict(base, vocab=97, width=40, streams=2, layers=[with_mlp(latent(2, 16, 8, 12, 20, base=100.0), None)])
    if which == "only_mlp_streams":   # the stream mixing and the feed-forward dominate: a tiny mixer, four streams
        return dict(base, vocab=97, width=40, streams=4, layers=[with_mlp(attention(1, 1, 8, 8, 3), 56), with_mlp(attention(1, 1, 8, 8, 3), 56)])
    if which == "odd":      # no size a multiple of 4: every kernel takes its scalar path, five streams, two taps
        return dict(base, vocab=61, width=50, streams=5, logit_softcap=9.0, loop=dict(start=1, stop=3, times=2), layers=[
            with_mlp(attention(3, 1, 10, 6, 5, 0.3), 70), with_mlp(mamba(30, 5, 2, 3), None),
            with_mlp(latent(2, 6, 6, 10, 14, base=300.0, dims=4), 34)])
    raise KeyError(which)


PAGE_SIZE = {"odd": 2, "mix": 16, "plain": 8, "one": 4, "only_mamba": 16, "only_attention": 8, "only_latent": 8, "only_mlp_streams": 16}


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> float32 tensor.  Matrices are drawn so that activations stay of order one through the layers, and
    what a recurrence or a softmax is sensitive to (step sizes, decays, sinks, mixing weights) covers a real range."""
    g = torch.Generator().manual_seed(seed)
    d, S = cfg["width"], cfg.get("streams")

    def mat(out, inp, gain=1.0):
        return torch.randn(out, inp, generator=g) * (gain / math.sqrt(inp))

    def uni(shape, a, b):
        return a + (b - a) * torch.rand(shape, generator=g)

    W = {"embed": torch.randn(cfg["vocab"], d, generator=g), "head": mat(cfg["vocab"], d, 2.0), "final.norm": uni((d,), 0.8, 1.2)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"] = uni((d,), 0.8, 1.2)
        if L["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = mat(H * dk, d, 2.0), mat(G * dk, d, 2.0), mat(G * dv, d)
            W[p + "mix.sink"] = uni((H,), -1.0, 2.0)
            W[p + "mix.o"] = mat(d, H * dv)
        elif L["type"] == "latent_attention":
            H, dk, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            W[p + "mix.q"], W[p + "mix.dkv"] = mat(H * (dk + dr), d, 2.0), mat(R + dr, d, 2.0)
            W[p + "mix.dkv.norm"] = uni((R,), 0.8, 1.2)
            W[p + "mix.uk"], W[p + "mix.uv"], W[p + "mix.o"] = mat(H * dk, R, 2.0), mat(H * dv, R), mat(d, H * dv)
        else:
            C, N, taps, r = m["inner"], m["state"], m["conv"], m["dt_rank"]
            W[p + "mix.in"] = mat(2 * C, d)
            W[p + "mix.conv"], W[p + "mix.conv.b"] = uni((C, taps), -0.6, 0.6), uni((C,), -0.2, 0.2)
            W[p + "mix.x"], W[p + "mix.dt"], W[p + "mix.dt.b"] = mat(r + 2 * N, C), mat(C, r), uni((C,), -4.0, 0.5)
            W[p + "mix.A_log"], W[p + "mix.D"], W[p + "mix.o"] = uni((C, N), -2.0, 1.5), uni((C,), 0.5, 1.5), mat(d, C)
        subs = ["hc1"]
        if L.get("mlp"):
            W[p + "norm2"] = uni((d,), 0.8, 1.2)
            W[p + "mlp.up"], W[p + "mlp.down"] = mat(L["mlp"]["ff"], d), mat(d, L["mlp"]["ff"])
            subs.append("hc2")
        if S:
            for hc in subs:
                W[p + hc + ".in"], W[p + hc + ".out"] = uni((S,), 0.1, 0.7), uni((S,), -1.0, 1.0)
                W[p + hc + ".mix"] = torch.eye(S) * 0.8 + uni((S, S), -0.2, 0.2)
    # every value is representable in bfloat16, so the 32-bit and the bfloat16 engine and the plain implementation
    # all hold the same weights
    return {k: v.to(torch.bfloat16).float() for k, v in W.items()}


def write_folder(root, name: str, cfg: dict, weights: dict) -> Path:
    from delta_b200.weights.safetensors_io import write_safetensors
    folder = Path(root) / name
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(folder / "model.safetensors", {k: v.contiguous() for k, v in weights.items()})
    return folder
