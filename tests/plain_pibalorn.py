"""A plain, slow implementation of the Pibalorn design in float64, one function per mechanism.

It shares no code with the engine: whole sequences at once, no cache, no pages, a loop over
tokens where a recurrence runs.  ``forward`` takes the dict of config.json, a dict
name -> tensor and the token ids of one sequence, and returns the logits of every position
and the residual stream after every layer run.

Notation: T tokens, d width, H heads, G key-value heads.
"""
from __future__ import annotations

import math

import torch

F = torch.float64

# With ``rounding("bfloat16")`` active every product's result and every activation between products is rounded to
# bfloat16 once, as a 16-bit engine does; what the design keeps in 32 bit is not.  By default nothing is rounded.
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
    return rnd(h @ w.to(F).T)


# ---------------------------------------------------------------- norms

def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    dev = x - mu
    var = (dev * dev).mean(-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * w.to(F)


# ------------------------------------------------------------ embedding

def embed_tokens(cfg, W, tokens):
    """Token rows times the scale, plus a row of the bigram table picked by a hash of (previous token, token); the
    first token of a sequence takes the table's last row."""
    e = cfg.get("embedding") or {}
    x = W["embed"].to(F)[tokens] * float(e.get("scale", 1.0))
    bg = e.get("bigram")
    if bg:
        n = int(bg["buckets"])
        rows = []
        for i, t in enumerate(tokens.tolist()):
            rows.append(n if i == 0 else (tokens[i - 1].item() * int(bg["mul_prev"]) + t * int(bg["mul_cur"])) % n)
        x = x + W["bigram"].to(F)[torch.tensor(rows)]
    return x


# ------------------------------------------------------------ attention

def rotate_half(x, positions, base, dims):
    """x [T, heads, n]: entry i of the first ``dims`` is paired with entry i + dims/2 and the pair turned by
    position * base^(-2i/dims)."""
    half = dims // 2
    freq = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = positions.to(F)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def attention(m, W, p, h, eps):
    """Grouped-query attention whose values are the keys as projected; rotated and unit-normed queries and keys;
    causal; a softmax with one more in its denominator."""
    T = h.shape[0]
    H, G, dk = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = lin(h, W[p + "q"]).view(T, H, dk)
    k = lin(h, W[p + "k"]).view(T, G, dk)
    v = k
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        q, k = rotate_half(q, pos, rot["base"], int(rot["dims"])), rotate_half(k, pos, rot["base"], int(rot["dims"]))
    q, k = rnd(unit_rms(q, eps)), rnd(unit_rms(k, eps))
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(pos[None, :] > pos[:, None], -math.inf)
        mx = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - mx)
        w = e / (torch.exp(-mx) + e.sum(-1, keepdim=True))
        out[:, hh] = w @ v[:, g]
    return lin(rnd(out.reshape(T, -1)), W[p + "o"])


# ---------------------------------------------------- lightning attention

def lightning(m, W, p, h, eps):
    """Linear attention with a constant decay per head: S <- decay S + k v^T, o = S^T q, token by token; the heads'
    outputs are normed together, gated and projected."""
    T = h.shape[0]
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    act = torch.nn.functional.silu
    q = rnd(act(lin(h, W[p + "q"]))).view(T, H, dk)
    k = rnd(act(lin(h, W[p + "k"]))).view(T, H, dk)
    v = rnd(act(lin(h, W[p + "v"]))).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        lam = float(m["decay"][hh])
        S = torch.zeros(dk, dv, dtype=F)
        for t in range(T):
            S = lam * S + torch.outer(k[t, hh], v[t, hh])
            out[t, hh] = S.T @ q[t, hh]
    o = unit_rms(out.reshape(T, H * dv), eps) * W[p + "norm"].to(F)
    o = rnd(o * torch.sigmoid(lin(h, W[p + "g"])))
    return lin(o, W[p + "o"])


# ------------------------------------------------------------ feed-forward

def glu(W, p, h, limit):
    g, u = lin(h, W[p + "gate"]), lin(h, W[p + "up"])
    if limit is not None:
        g, u = torch.clamp(g, max=float(limit)), torch.clamp(u, min=-float(limit), max=float(limit))
    y = rnd(g * torch.sigmoid(1.702 * g) * (u + 1.0))
    return lin(y, W[p + "down"])


def experts(mlp, W, p, h):
    T = h.shape[0]
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ W[p + "router"].to(F).T
    vals, idx = torch.topk(z, top, dim=-1)
    w = torch.softmax(vals, dim=-1)
    out = torch.zeros(T, h.shape[1], dtype=F)
    for t in range(T):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += w[t, j] * glu(W, f"{p}e{e}.", h[t:t + 1], mlp["expert"].get("limit"))[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ W[p + "shared.sg"].to(F).T)
        out = out + gate * glu(W, p + "shared.", h, mlp["shared"].get("limit"))
    return rnd(out)


def feed_forward(mlp, W, p, h):
    if mlp["kind"] == "dense":
        return glu(W, p, h, mlp.get("limit"))
    if mlp["kind"] == "moe":
        return experts(mlp, W, p, h)
    raise ValueError(mlp["kind"])


# ----------------------------------------------------------------- model

def run_order(cfg):
    """[(layer, number of the pass this run starts, or None)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(cfg, W, tokens):
    """tokens: LongTensor [T].  Returns (logits [T, vocab], residual stream after every layer run [runs, T, d])."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = float(cfg["norm"]["eps"])
    x0 = embed_tokens(cfg, W, tokens)
    x = x0.clone()
    after = []
    for i, enters in run_order(cfg):
        if enters is not None:
            if enters > 0:
                x = x + x0
            x = x + W["loop.step"].to(F)[enters]
        L = cfg["layers"][i]
        p = f"l{i}."
        h = rnd(layer_norm(x, W[p + "norm1"], eps))
        mix = attention(L["mixer"], W, p + "mix.", h, eps) if L["type"] == "attention" else lightning(L["mixer"], W, p + "mix.", h, eps)
        if L.get("mlp"):
            mix = mix + feed_forward(L["mlp"], W, p + "mlp.", h)
        x = x + mix
        after.append(x.clone())
    hN = rnd(layer_norm(x, W["final.norm"], eps))
    return hN @ W["head"].to(F).T, torch.stack(after)
