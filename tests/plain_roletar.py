"""A plain, slow implementation of the Roletar design in float64, one function per mechanism.

It shares no code with the engine: whole sequences at once, no cache, no pages, loops
over tokens where a recurrence runs.  ``forward`` takes the dict of config.json and a dict
name -> tensor and returns the logits of every position and the summed residual streams
after every layer run.

Notation: T tokens, d width, S residual streams, H heads.
"""
from __future__ import annotations

import math

import torch

F = torch.float64

# What a 16-bit engine rounds: with ``rounding("bfloat16")`` active, every product's result and every activation between
# products is rounded to bfloat16 once (and carried on in float64); what the design computes in 32 bit (the residual
# streams, norms' statistics, scores and softmax weights, step sizes, decays, states) is not.  By default nothing is rounded.
_round = [lambda x: x]


class rounding:
    def __init__(self, kind):
        self.fn = (lambda x: x.to(torch.bfloat16).to(F)) if kind == "bfloat16" else (lambda x: x)

    def __enter__(self):
        self.old = _round[0]
        _round[0] = self.fn

    def __exit__(self, *a):
        _round[0] = self.old


def rnd(x):
    return _round[0](x)


def lin(h, w):
    """h W^T, the result rounded as an engine's product would be."""
    return rnd(h @ w.T)


def rms_unit(x, eps):
    """x scaled to unit root mean square over its last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def rotate_pairs(x, positions, base, dims):
    """Rotary positions on the first ``dims`` entries of the last axis of x [T, ..., n]; entries
    2i and 2i+1 form pair i, turned by the angle position * base^(-2i/dims)."""
    T = x.shape[0]
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = positions.to(F)[:, None] * freq[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [half]
    cos, sin = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def softmax_rows(scores, visible, sink=None):
    """Softmax over the visible keys of every query row of scores [T, T]; ``sink`` adds exp(sink) to the
    denominator and nothing to the numerator."""
    s = scores.masked_fill(~visible, -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, torch.full_like(m, float(sink)))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink - m)
    return e / den


def causal_mask(T, window=None):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    vis = j <= i
    if window is not None:
        vis &= (i - j) < window
    return vis


def windowed_sink_attention(h, W, pre, m):
    """Grouped-query attention without positions: sliding window, a per-head sink in the softmax."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = lin(h, W[pre + "q"]).view(T, H, dk)
    k = lin(h, W[pre + "k"]).view(T, G, dk)
    v = lin(h, W[pre + "v"]).view(T, G, dv)
    window = m["mask"]["size"] if m.get("mask") else None
    vis = causal_mask(T, window)
    out = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        sc = (q[:, hh] @ k[:, g].T) * m["scale"]
        p = softmax_rows(sc, vis, W[pre + "sink"][hh])
        out[:, hh] = p @ v[:, g]
    return lin(rnd(out.reshape(T, H * dv)), W[pre + "o"])


def latent_attention(h, W, pre, m, eps):
    """Attention over a shared low-rank latent: keys and values of every head are products of one
    normalised latent vector per token; a small rotated key part is shared by all heads."""
    T = h.shape[0]
    H, dk, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = lin(h, W[pre + "q"]).view(T, H, dk + dr)
    q_plain, q_rot = q[..., :dk], q[..., dk:]
    low = lin(h, W[pre + "dkv"])
    c = rnd(rms_norm(low[:, :R], W[pre + "dkv.norm"], eps))
    k_rot = low[:, R:]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q_rot = rnd(rotate_pairs(q_rot, pos, base, dims))
    k_rot = rnd(rotate_pairs(k_rot, pos, base, dims))
    k_plain = lin(c, W[pre + "uk"]).view(T, H, dk)
    v = lin(c, W[pre + "uv"]).view(T, H, dv)
    vis = causal_mask(T)
    out = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        sc = (q_plain[:, hh] @ k_plain[:, hh].T + q_rot[:, hh] @ k_rot.T) * m["scale"]
        out[:, hh] = softmax_rows(sc, vis) @ v[:, hh]
    return lin(rnd(out.reshape(T, H * dv)), W[pre + "o"])


def silu(x):
    return x / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def selective_scan_mixer(h, W, pre, m):
    """Selective state-space mixer: short causal convolution, input-dependent step size, diagonal decay."""
    T = h.shape[0]
    C_, N, taps, rank = m["inner"], m["state"], m["conv"], m["dt_rank"]
    xz = lin(h, W[pre + "in"])
    x, z = xz[:, :C_], xz[:, C_:]
    padded = torch.cat([torch.zeros(taps - 1, C_, dtype=F), x], 0)
    conv = torch.zeros(T, C_, dtype=F)
    for j in range(taps):          # column taps-1 multiplies the current token
        conv += padded[j:j + T] * W[pre + "conv"][:, j][None, :]
    x = rnd(silu(conv + W[pre + "conv.b"][None, :]))
    low = lin(x, W[pre + "x"])
    dt = softplus(lin(low[:, :rank], W[pre + "dt"]) + W[pre + "dt.b"][None, :])
    Bm, Cm = low[:, rank:rank + N], low[:, rank + N:rank + 2 * N]
    A = -torch.exp(W[pre + "A_log"])
    state = torch.zeros(C_, N, dtype=F)
    y = torch.zeros(T, C_, dtype=F)
    for t in range(T):
        state = torch.exp(dt[t][:, None] * A) * state + (dt[t] * x[t])[:, None] * Bm[t][None, :]
        y[t] = state @ Cm[t] + W[pre + "D"] * x[t]
    return lin(rnd(y * silu(z)), W[pre + "o"])


def dense_ff(h, W, pre):
    a = torch.relu(lin(h, W[pre + "up"]))
    return lin(rnd(a * a), W[pre + "down"])


def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def mixer_of(layer, h, W, pre, eps):
    kind, m = layer["type"], layer["mixer"]
    if kind == "attention":
        return windowed_sink_attention(h, W, pre, m)
    if kind == "latent_attention":
        return latent_attention(h, W, pre, m, eps)
    if kind == "mamba1":
        return selective_scan_mixer(h, W, pre, m)
    raise KeyError(kind)


def forward(cfg, weights, tokens):
    """logits [T, vocab] and the summed streams after every layer run [runs, T, d], float64."""
    W = {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    S = cfg.get("streams")
    x0 = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    X = [x0.clone() for _ in range(S or 1)]
    after = []
    for li in order_of(cfg):
        layer = cfg["layers"][li]
        subs = [("hc1", "norm1", lambda h, li=li, layer=layer: mixer_of(layer, h, W, f"l{li}.mix.", eps))]
        if layer.get("mlp"):
            subs.append(("hc2", "norm2", lambda h, li=li: dense_ff(h, W, f"l{li}.mlp.")))
        for hc, norm, fn in subs:
            if S:
                w_in, w_out, w_mix = W[f"l{li}.{hc}.in"], W[f"l{li}.{hc}.out"], W[f"l{li}.{hc}.mix"]
                u = sum(w_in[s] * X[s] for s in range(S))
                y = fn(rnd(rms_norm(u, W[f"l{li}.{norm}"], eps)))
                X = [sum(w_mix[s, t] * X[s] for s in range(S)) + w_out[t] * y for t in range(S)]
            else:
                X = [X[0] + fn(rnd(rms_norm(X[0], W[f"l{li}.{norm}"], eps)))]
        after.append(sum(X))
    x = sum(X)
    logits = rnd(rms_norm(x, W["final.norm"], eps)) @ W["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, torch.stack(after)


order_of = run_order
