"""Roletar as a ``ModelSpec``: a decoder whose layers are listed in config.json, each with one of three mixers
(windowed grouped-query attention with a softmax sink, latent attention, a selective state-space mixer) and an
optional dense feed-forward with a squared-relu activation; a 32-bit residual stream kept as several mixed
copies; a span of layers that runs several times with the same weights, every run with a cache or state of its
own; soft-capped logits.

Tensor names: ``embed``, ``head``, ``final.norm``; layer i: ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.up|down``, ``l<i>.hc1.*`` and ``l<i>.hc2.*`` (the stream mixing of the two sublayers).
"""
from __future__ import annotations

from typing import Optional

from ..config.engine_config import EngineConfig
from ..config.roletar_config import RoletarConfig
from ..parts.base import PartSpec, TensorSpec
from .spec import LayerSpec, ModelSpec, RunEntry


def _mixer(cfg: RoletarConfig, i: int, max_pos: int) -> PartSpec:
    L = cfg.layers[i]
    m, pre, d = L.mixer, f"l{i}.mix.", cfg.width
    if L.type == "attention":
        mask = m.get("mask") or {}
        return PartSpec("sink_attention", dict(prefix=pre, width=d, heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"],
                                               value_dim=m["vdim"], window=mask.get("size"), sink=True, scale=m["scale"]), "mixer")
    if L.type == "latent_attention":
        position = None
        if m["rot_dim"]:
            position = PartSpec("rotary", dict(head_dim=m["rot"]["dims"], theta=m["rot"]["base"], max_positions=max_pos,
                                               interleaved=True), "position")
        return PartSpec("latent_attention", dict(prefix=pre, width=d, heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"],
                                                 value_dim=m["vdim"], kv_rank=m["kv_rank"], eps=cfg.eps, scale=m["scale"],
                                                 position=position, rot_dims=m["rot"]["dims"] if m["rot_dim"] else None), "mixer")
    return PartSpec("selective_scan", dict(prefix=pre, width=d, inner=m["inner"], state=m["state"], conv=m["conv"],
                                           dt_rank=m["dt_rank"]), "mixer")


def roletar_spec(cfg: RoletarConfig, engine: Optional[EngineConfig] = None) -> ModelSpec:
    engine = engine or EngineConfig()
    d, S = cfg.width, cfg.streams
    layers = []
    for i, L in enumerate(cfg.layers):
        pre = f"l{i}."

        def mixing(q, pre=pre):
            return PartSpec("learned", dict(copies=S or 1, prefix=(pre + f"hc{q}.") if S else None), "stream_mixing")

        parts = dict(norm1=PartSpec("rms_norm", dict(name=pre + "norm1", width=d, eps=cfg.eps), "norm"),
                     mixer=_mixer(cfg, i, engine.max_seq_len), mixing1=mixing(1))
        if L.mlp is not None:
            parts.update(norm2=PartSpec("rms_norm", dict(name=pre + "norm2", width=d, eps=cfg.eps), "norm"),
                         feed_forward=PartSpec("dense_mlp", dict(prefix=pre + "mlp.", width=d, intermediate=L.mlp["ff"],
                                                                 activation="relu2"), "feed_forward"),
                         mixing2=mixing(2))
        layers.append(LayerSpec(parts, block="stream_pre_norm"))
    return ModelSpec(
        vocab_size=cfg.vocab, width=d, layers=tuple(layers), order=tuple(RunEntry(i) for i in cfg.run_order()),
        final_norm=PartSpec("rms_norm", dict(name="final.norm", width=d, eps=cfg.eps), "norm"),
        embedding=TensorSpec("embed", (cfg.vocab, d), kind="table"), lm_head=TensorSpec("head", (cfg.vocab, d), kind="matrix"),
        max_positions=engine.max_seq_len, stream=PartSpec("mixed_f32", dict(width=d, copies=S or 1), "stream"),
        logit_softcap=cfg.logit_softcap)
