"""Pibalorn as a ``ModelSpec``: a decoder whose layers are listed in config.json.  Every layer is a parallel block (one
layer norm without bias; the mixer and the feed-forward both read it and their outputs are summed into a 32-bit
residual stream) with one of two mixers: grouped-query attention whose values are its keys as projected, with partly
rotated, unit-normed queries and keys and one more in the softmax's denominator; or linear attention with a constant
decay per head and a gated norm.  The feed-forward is a gated one with clamped branches, dense or as a mixture of experts
with a shared expert.  The embedding is scaled and gets a hashed pair ("bigram") table added; a span of layers may run
several times with the same weights, every run with a cache or state of its own, the embedding output and a vector per
pass being added when a pass starts.

Tensor names: ``embed``, ``bigram``, ``loop.step``, ``head``, ``final.norm``; layer i: ``l<i>.norm1``, ``l<i>.mix.*``,
``l<i>.mlp.*``.
"""
from __future__ import annotations

from typing import Optional

from ..config.engine_config import EngineConfig
from ..config.pibalorn_config import PibalornConfig
from ..parts.base import PartSpec, TensorSpec
from .spec import LayerSpec, ModelSpec, RunEntry

GLU_ALPHA = 1.702     # the design fixes  y = g sigmoid(1.702 g) (u + 1)
GLU_SHIFT = 1.0
SINK_LOGIT = 0.0      # one more in the softmax's denominator: a sink whose logit is 0


def _mixer(cfg: PibalornConfig, i: int, max_pos: int) -> PartSpec:
    L = cfg.layers[i]
    m, pre, d = L.mixer, f"l{i}.mix.", cfg.width
    if L.type == "attention":
        rot = m.get("rot") or None
        position = None
        if rot and rot["dims"]:
            position = PartSpec("rotary", dict(head_dim=rot["dims"], theta=rot["base"], max_positions=max_pos, interleaved=False), "position")
        return PartSpec("sink_attention", dict(prefix=pre, width=d, heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"],
                                               value_dim=m["vdim"], scale=m["scale"], position=position,
                                               rot_dims=rot["dims"] if position is not None else None, sink_logit=SINK_LOGIT,
                                               unit_norm_eps=cfg.eps, value_from_key=True), "mixer")
    return PartSpec("decay_attention", dict(prefix=pre, width=d, heads=m["heads"], head_dim=m["dim"], value_dim=m["vdim"],
                                            decays=tuple(m["decay"]), eps=cfg.eps), "mixer")


def _feed_forward(cfg: PibalornConfig, i: int) -> Optional[PartSpec]:
    mlp, pre, d = cfg.layers[i].mlp, f"l{i}.mlp.", cfg.width
    if mlp is None:
        return None
    glu = dict(alpha=GLU_ALPHA, shift=GLU_SHIFT)
    if mlp["kind"] == "dense":
        return PartSpec("clamped_glu", dict(prefix=pre, width=d, intermediate=mlp["ff"], limit=mlp.get("limit"), **glu), "feed_forward")
    shared = mlp.get("shared")
    return PartSpec("experts", dict(prefix=pre, width=d, experts=mlp["router"]["experts"], top=mlp["router"]["top"],
                                    intermediate=mlp["expert"]["ff"], limit=mlp["expert"].get("limit"),
                                    shared=dict(intermediate=shared["ff"], limit=shared.get("limit")) if shared else None, **glu),
                    "feed_forward")


def pibalorn_spec(cfg: PibalornConfig, engine: Optional[EngineConfig] = None) -> ModelSpec:
    engine = engine or EngineConfig()
    d = cfg.width
    layers = []
    for i in range(len(cfg.layers)):
        parts = dict(norm1=PartSpec("layer_norm", dict(name=f"l{i}.norm1", width=d, eps=cfg.eps), "norm"),
                     mixer=_mixer(cfg, i, engine.max_seq_len))
        ff = _feed_forward(cfg, i)
        if ff is not None:
            parts["feed_forward"] = ff
        layers.append(LayerSpec(parts, block="parallel"))
    pair = dict(cfg.bigram, name="bigram") if cfg.bigram else None
    reentry = dict(name="loop.step", passes=cfg.loop["times"], add_embedding=True) if cfg.loop else None
    return ModelSpec(
        vocab_size=cfg.vocab, width=d, layers=tuple(layers),
        order=tuple(RunEntry(i, enters_pass=t) for i, t in cfg.run_order()),
        final_norm=PartSpec("layer_norm", dict(name="final.norm", width=d, eps=cfg.eps), "norm"),
        embedding=TensorSpec("embed", (cfg.vocab, d), kind="table"), lm_head=TensorSpec("head", (cfg.vocab, d), kind="matrix"),
        max_positions=engine.max_seq_len,
        stream=PartSpec("residual_f32", dict(width=d, scale=cfg.embed_scale, pair=pair, reentry=reentry), "stream"))
