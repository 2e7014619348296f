"""Pibalorn on the CPU: the configuration reader, the run order, the specification's tensor list against the names the
tests write out on their own, and properties of the plain implementation that the GPU tests lean on."""
import math

import pytest
import torch

import pibalorn_helpers as ph
import plain_pibalorn as plain

ALL = ["wide", "mix", "odd", "one", "sharp", "only_attention", "only_lightning", "only_experts", "only_pairs", "pairs_many"]


def build(which):
    import delta_b200.models  # noqa: F401
    from delta_b200.config.registry import architecture_of
    from delta_b200.models import Model
    cfg = ph.config(which)
    arch = architecture_of(cfg)
    typed = arch.config_from_dict(cfg)
    return cfg, typed, Model(arch.build_spec(typed, None))


@pytest.mark.parametrize("which", ALL)
def test_tensor_list(which):
    cfg, typed, model = build(which)
    want = {k: tuple(v.shape) for k, v in ph.make_weights(cfg, 1).items()}
    got = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert got == want


def test_run_order_and_passes():
    cfg, typed, model = build("mix")
    assert typed.run_order() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert typed.run_order() == plain.run_order(cfg)
    assert [e.enters_pass for e in model.order] == [None, 0, None, 1, None, None]
    assert len({e.cache for e in model.order}) == 6        # every run has a cache or state of its own
    cfg, typed, model = build("odd")
    assert [e.enters_pass for e in model.order] == [0, None, 1, None, 2, None, None]
    cfg, typed, model = build("only_attention")
    assert [e.enters_pass for e in model.order] == [None]
    with pytest.raises(NotImplementedError):
        from delta_b200.parts.base import Stream
        Stream().enter_pass(None, None, None, 0)


def test_state_and_cache_declared_per_run():
    cfg, typed, model = build("mix")
    states = model.state_specs()
    assert "stream.prev_token" in states and states["stream.prev_token"].dtype == torch.int32 and states["stream.prev_token"].fill == -1
    runs = sorted(k for k in states if k.startswith("run"))
    assert runs == ["run0.decay_attention", "run2.decay_attention", "run4.decay_attention"]
    assert states["run2.decay_attention"].shape == (2, 24, 16)
    assert sorted(model.cache_specs()) == [1, 3, 5]
    assert model.has_run_state()
    cfg, typed, model = build("sharp")           # no recurrent layer and no pair table: nothing is carried but pages
    assert not model.has_run_state() and not model.state_specs()
    cfg, typed, model = build("only_pairs")      # the previous token alone makes a step one that cannot be run twice
    assert model.has_run_state()


def test_config_errors():
    from delta_b200.config.model_config import ConfigError
    from delta_b200.config.pibalorn_config import PibalornConfig
    good = ph.config("mix")
    PibalornConfig.from_dict(good)
    for path, value, text in ((("layers", 1, "mixer", "vdim"), 20, "vdim"), (("layers", 1, "mixer", "kv_heads"), 3, "multiple"),
                              (("layers", 0, "mixer", "decay"), [0.5], "decays"), (("loop", "stop"), 9, "loop"),
                              (("layers", 1, "mlp", "router", "top"), 7, "top"), (("layers", 1, "mixer", "rot", "dims"), 15, "rot.dims"),
                              (("layers", 0, "type"), "mamba", "unknown mixer"), (("layers", 0, "mlp", "kind"), "glu", "feed-forward kind")):
        import copy
        bad = copy.deepcopy(good)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=text):
            PibalornConfig.from_dict(bad)
    for key in ("vocab", "width", "norm", "layers"):
        bad = {k: v for k, v in good.items() if k != key}
        with pytest.raises(ConfigError, match=key):
            PibalornConfig.from_dict(bad)


def test_plain_pair_rows_and_first_token():
    cfg = ph.config("pairs_many")
    W = ph.make_weights(cfg, 3)
    toks = torch.tensor([249, 249, 7, 0])
    x = plain.embed_tokens(cfg, W, toks)
    bg = cfg["embedding"]["bigram"]
    row = (249 * bg["mul_prev"] + 249 * bg["mul_cur"]) % bg["buckets"]
    assert 249 * bg["mul_prev"] + 249 * bg["mul_cur"] < 2 ** 31 < 249 * bg["mul_prev"] * 100      # near the edge of 32 bits
    assert torch.allclose(x[0], W["embed"][249].double() + W["bigram"][bg["buckets"]].double())
    assert torch.allclose(x[1], W["embed"][249].double() + W["bigram"][row].double())


def test_plain_sink_and_decay():
    """The softmax's extra one: a lone first token attends to itself with weight e^s / (1 + e^s), not 1; and linear
    attention's second output mixes the first key-value pair scaled by the decay."""
    cfg = ph.config("only_attention")
    W = ph.make_weights(cfg, 5)
    m = cfg["layers"][0]["mixer"]
    h = torch.randn(1, cfg["width"], dtype=torch.float64)
    out = plain.attention(m, W, "l0.mix.", h, 1e-5)
    k = (h @ W["l0.mix.k"].double().T).view(m["kv_heads"], m["dim"])
    q = (h @ W["l0.mix.q"].double().T).view(m["heads"], m["dim"])
    want = []
    for hh in range(m["heads"]):
        g = hh // (m["heads"] // m["kv_heads"])
        s = (plain.unit_rms(q[hh], 1e-5) @ plain.unit_rms(k[g], 1e-5)) * m["scale"]     # position 0: no rotation
        want.append(torch.exp(s) / (1 + torch.exp(s)) * k[g])
    assert torch.allclose(out[0], torch.cat(want) @ W["l0.mix.o"].double().T)
    cfg = ph.config("only_lightning")
    W = ph.make_weights(cfg, 6)
    m = cfg["layers"][0]["mixer"]
    h = torch.randn(2, cfg["width"], dtype=torch.float64)
    act = torch.nn.functional.silu
    q, k, v = (act(h @ W["l0.mix." + n].double().T) for n in "qkv")
    o = []
    for hh, lam in enumerate(m["decay"]):
        a, b = slice(hh * m["dim"], (hh + 1) * m["dim"]), slice(hh * m["vdim"], (hh + 1) * m["vdim"])
        o.append(lam * (q[1, a] @ k[0, a]) * v[0, b] + (q[1, a] @ k[1, a]) * v[1, b])
    o = torch.cat(o)
    y = plain.unit_rms(o, 1e-5) * W["l0.mix.norm"].double() * torch.sigmoid(h[1] @ W["l0.mix.g"].double().T)
    assert torch.allclose(plain.lightning(m, W, "l0.mix.", h, 1e-5)[1], y @ W["l0.mix.o"].double().T)
