"""Typed configuration of the Roletar design, read from its config.json.

The file names the design in ``architecture`` and gives every size and every constant that may differ between
models of the design:

    vocab, width                      token interface and stream width
    norm.eps                          eps of every RMSNorm
    streams                           copies of the residual stream (absent: one copy, the plain residual sum)
    logit_softcap                     logits <- cap * tanh(logits / cap) (absent: none)
    loop {start, stop, times}         layers start..stop-1 run ``times`` times in a row with the same weights
    layers[i] {type, mixer, mlp}      the mixer's kind and sizes; mlp {kind, ff} or null

Mixer kinds and their keys:
    attention          heads, kv_heads, dim, vdim, scale, mask.size (the sliding window)
    latent_attention   heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}
    mamba1             inner, state, conv, dt_rank
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .model_config import ConfigError

MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"),
    "mamba1": ("inner", "state", "conv", "dt_rank"),
}


@dataclass(frozen=True)
class RoletarLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]


@dataclass(frozen=True)
class RoletarConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: tuple
    streams: Optional[int] = None
    logit_softcap: Optional[float] = None
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def from_dict(c: dict) -> "RoletarConfig":
        def need(d, key, where):
            if not isinstance(d, dict) or key not in d or d[key] is None:
                raise ConfigError(f"config.json has no '{key}' in {where}")
            return d[key]

        layers = []
        raw_layers = need(c, "layers", "the model")
        if not raw_layers:
            raise ConfigError("config.json lists no layers")
        for i, L in enumerate(raw_layers):
            kind = need(L, "type", f"layer {i}")
            if kind not in MIXER_KEYS:
                raise ConfigError(f"layer {i}: unknown mixer type '{kind}'; known: {', '.join(MIXER_KEYS)}")
            m = dict(need(L, "mixer", f"layer {i}"))
            for k in MIXER_KEYS[kind]:
                need(m, k, f"the mixer of layer {i}")
            if kind == "latent_attention" and m["rot_dim"]:
                rot = need(m, "rot", f"the mixer of layer {i}")
                need(rot, "base", f"rot of layer {i}")
                need(rot, "dims", f"rot of layer {i}")
            if kind == "attention" and m.get("mask") is not None:
                need(m["mask"], "size", f"mask of layer {i}")
            mlp = L.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"layer {i}: unknown feed-forward kind '{mlp.get('kind')}' (dense only)")
                need(mlp, "ff", f"mlp of layer {i}")
                mlp = dict(mlp)
            layers.append(RoletarLayer(kind, m, mlp))
        loop = c.get("loop") or {}
        cfg = RoletarConfig(
            architecture=str(c.get("architecture") or (c.get("architectures") or ["Roletar"])[0]),
            vocab=int(need(c, "vocab", "the model")), width=int(need(c, "width", "the model")),
            eps=float(need(need(c, "norm", "the model"), "eps", "norm")), layers=tuple(layers),
            streams=int(c["streams"]) if c.get("streams") is not None else None,
            logit_softcap=float(c["logit_softcap"]) if c.get("logit_softcap") else None,
            loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)), loop_times=int(loop.get("times", 1)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1:
            raise ConfigError("vocab and width must be positive")
        if self.streams is not None and not (1 <= self.streams <= 8):
            raise ConfigError(f"streams must be 1 to 8, got {self.streams}")
        n = len(self.layers)
        if not (0 <= self.loop_start <= self.loop_stop <= n) or self.loop_times < 1:
            raise ConfigError(f"loop {self.loop_start}..{self.loop_stop} x {self.loop_times} does not fit {n} layers")
        for i, L in enumerate(self.layers):
            m = L.mixer
            if L.type == "attention" and m["heads"] % m["kv_heads"]:
                raise ConfigError(f"layer {i}: {m['heads']} heads are no multiple of {m['kv_heads']} key-value heads")
            if L.type == "latent_attention" and m["rot_dim"] and (m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["rot_dim"]):
                raise ConfigError(f"layer {i}: rot.dims {m['rot']['dims']} must be even and at most rot_dim {m['rot_dim']}")

    def run_order(self) -> list:
        """Layer indices in the order they run: the looped span repeated in place."""
        a, b = self.loop_start, self.loop_stop
        return list(range(a)) + list(range(a, b)) * self.loop_times + list(range(b, len(self.layers)))
