"""Typed configuration of the Pibalorn design, read from its config.json.

The file names the design in ``architecture`` and gives every size and every constant that may differ between
models of the design:

    vocab, width                         token interface and stream width
    norm.eps                             eps of every norm (layer norms, the unit norms of queries and keys, the gated norm)
    embedding.scale                      factor on the token embedding
    embedding.bigram {buckets, mul_prev, mul_cur}   the hashed pair table (absent: none)
    loop {start, stop, times}            layers start..stop-1 run ``times`` times in a row with the same weights (absent: none)
    layers[i] {type, mixer, mlp}         the mixer's kind and sizes; mlp or null

Mixer kinds and their keys:
    attention   heads, kv_heads, dim, vdim, scale, rot {base, dims} (absent: no rotation)
    lightning   heads, dim, vdim, decay [heads]
Feed-forward kinds:
    dense       ff, limit
    moe         router {experts, top}, expert {ff, limit}, shared {ff, limit} (absent: no shared expert)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .model_config import ConfigError

MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "lightning": ("heads", "dim", "vdim", "decay"),
}


@dataclass(frozen=True)
class PibalornLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]


@dataclass(frozen=True)
class PibalornConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: tuple
    embed_scale: float = 1.0
    bigram: Optional[dict] = None
    loop: Optional[dict] = None

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def from_dict(c: dict) -> "PibalornConfig":
        def need(d, key, where):
            if not isinstance(d, dict) or key not in d or d[key] is None:
                raise ConfigError(f"config.json has no '{key}' in {where}")
            return d[key]

        raw_layers = need(c, "layers", "the model")
        if not raw_layers:
            raise ConfigError("config.json lists no layers")
        layers = []
        for i, L in enumerate(raw_layers):
            kind = need(L, "type", f"layer {i}")
            if kind not in MIXER_KEYS:
                raise ConfigError(f"layer {i}: unknown mixer type '{kind}'; known: {', '.join(MIXER_KEYS)}")
            m = dict(need(L, "mixer", f"layer {i}"))
            for k in MIXER_KEYS[kind]:
                need(m, k, f"the mixer of layer {i}")
            if kind == "attention" and m.get("rot"):
                need(m["rot"], "base", f"rot of layer {i}")
                need(m["rot"], "dims", f"rot of layer {i}")
            mlp = L.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                mk = need(mlp, "kind", f"mlp of layer {i}")
                if mk == "dense":
                    need(mlp, "ff", f"mlp of layer {i}")
                elif mk == "moe":
                    r = need(mlp, "router", f"mlp of layer {i}")
                    need(r, "experts", f"router of layer {i}")
                    need(r, "top", f"router of layer {i}")
                    need(need(mlp, "expert", f"mlp of layer {i}"), "ff", f"expert of layer {i}")
                    if mlp.get("shared"):
                        need(mlp["shared"], "ff", f"shared expert of layer {i}")
                else:
                    raise ConfigError(f"layer {i}: unknown feed-forward kind '{mk}' (dense, moe)")
            layers.append(PibalornLayer(kind, m, mlp))
        emb = c.get("embedding") or {}
        bigram = emb.get("bigram")
        if bigram:
            bigram = dict(buckets=int(need(bigram, "buckets", "embedding.bigram")), mul_prev=int(need(bigram, "mul_prev", "embedding.bigram")),
                          mul_cur=int(need(bigram, "mul_cur", "embedding.bigram")))
        loop = c.get("loop")
        if loop:
            loop = dict(start=int(need(loop, "start", "loop")), stop=int(need(loop, "stop", "loop")), times=int(need(loop, "times", "loop")))
        cfg = PibalornConfig(
            architecture=str(c.get("architecture") or (c.get("architectures") or ["Pibalorn"])[0]),
            vocab=int(need(c, "vocab", "the model")), width=int(need(c, "width", "the model")),
            eps=float(need(need(c, "norm", "the model"), "eps", "norm")), layers=tuple(layers),
            embed_scale=float(emb.get("scale", 1.0)), bigram=bigram or None, loop=loop or None)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1:
            raise ConfigError("vocab and width must be positive")
        if self.bigram and self.bigram["buckets"] < 1:
            raise ConfigError("embedding.bigram.buckets must be positive")
        n = len(self.layers)
        if self.loop:
            a, b, t = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not (0 <= a < b <= n) or t < 1:
                raise ConfigError(f"loop {a}..{b} x {t} does not fit {n} layers")
        for i, L in enumerate(self.layers):
            m = L.mixer
            if L.type == "attention":
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"layer {i}: {m['heads']} heads are no multiple of {m['kv_heads']} key-value heads")
                if m["vdim"] != m["dim"]:
                    raise ConfigError(f"layer {i}: the values are the keys, so vdim {m['vdim']} must equal dim {m['dim']}")
                rot = m.get("rot")
                if rot and (rot["dims"] % 2 or rot["dims"] > m["dim"]):
                    raise ConfigError(f"layer {i}: rot.dims {rot['dims']} must be even and at most dim {m['dim']}")
            else:
                if len(m["decay"]) != m["heads"]:
                    raise ConfigError(f"layer {i}: {len(m['decay'])} decays for {m['heads']} heads")
            if L.mlp and L.mlp["kind"] == "moe" and not (1 <= L.mlp["router"]["top"] <= L.mlp["router"]["experts"]):
                raise ConfigError(f"layer {i}: top {L.mlp['router']['top']} of {L.mlp['router']['experts']} experts")

    def run_order(self) -> list:
        """[(layer, number of the pass this run starts, or None)] in the order the layers run."""
        n = len(self.layers)
        if not self.loop:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order = [(i, None) for i in range(a)]
        for t in range(times):
            order += [(i, t if i == a else None) for i in range(a, b)]
        return order + [(i, None) for i in range(b, n)]
