"""Roletar without a GPU: the configuration reader, the run order, the model's tensor list, cache groups and
per-run state, and the plain implementation's own consistency."""
import json

import pytest
import torch

import plain_roletar as plain
import roletar_helpers as rh
from delta_b200.config import EngineConfig
from delta_b200.config.model_config import ConfigError
from delta_b200.config.registry import architecture_of
from delta_b200.models.model import Model

ALL = ["mix", "plain", "one", "odd", "only_mamba", "only_attention", "only_latent", "only_mlp_streams"]


def build(which, **engine):
    cfg_json = rh.config(which)
    arch = architecture_of(cfg_json)
    cfg = arch.config_from_dict(cfg_json)
    return cfg, Model(arch.build_spec(cfg, EngineConfig(**engine)))


@pytest.mark.parametrize("which", ALL)
def test_tensor_list_is_the_folder_layout(which):
    cfg, model = build(which)
    weights = rh.make_weights(rh.config(which), 0)
    specs = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert specs == {k: tuple(v.shape) for k, v in weights.items()}


def test_run_order_and_state_per_run():
    cfg, model = build("mix")
    assert cfg.run_order() == [0, 1, 0, 1, 2] == plain.run_order(rh.config("mix"))
    assert [e.layer for e in model.order] == [0, 1, 0, 1, 2]
    assert len({e.cache for e in model.order}) == 5            # every run has a cache or state of its own
    states = model.state_specs()
    assert sorted(states) == ["run0.conv", "run0.scan", "run2.conv", "run2.scan"]
    assert states["run0.scan"].shape == (160, 12) and states["run0.conv"].shape == (2, 160)
    specs = model.cache_specs()
    assert sorted(specs) == [1, 3, 4]
    assert specs[1] == specs[3] and specs[1].window == 21 and specs[4].window is None
    assert model.has_run_state()
    cfg, model = build("one")
    assert cfg.run_order() == [0, 1, 1, 1, 2]
    cfg, model = build("only_attention")
    assert not model.has_run_state()


def test_absent_keys_mean_absent_mechanisms():
    cfg, model = build("plain")
    assert cfg.streams is None and cfg.logit_softcap is None and cfg.run_order() == [0, 1, 2, 3]
    assert model.spec.logit_softcap is None and model.stream.copies == 1
    assert not any("hc" in s.name for s in model.tensor_specs())
    assert model.cache_specs()[3].window is None


def test_config_errors_name_the_key():
    c = rh.config("mix")
    del c["layers"][1]["mixer"]["kv_heads"]
    with pytest.raises(ConfigError, match="kv_heads"):
        architecture_of(c).config_from_dict(c)
    c = rh.config("mix")
    c["layers"][0]["type"] = "mamba7"
    with pytest.raises(ConfigError, match="mamba7"):
        architecture_of(c).config_from_dict(c)
    c = rh.config("mix")
    c["loop"]["stop"] = 9
    with pytest.raises(ConfigError, match="loop"):
        architecture_of(c).config_from_dict(c)


def test_cache_manager_and_scheduler_take_a_model_without_pages():
    """A model of recurrent layers only has no cache group; slots and state still work."""
    from delta_b200.cache.manager import CacheManager
    from delta_b200.engine.scheduler import Scheduler
    cfg, model = build("only_mamba")
    cm = CacheManager(model.cache_specs(), model.state_specs(), max_slots=2, max_seq_len=64, page_size=16, num_pages=8,
                      dtype=torch.float32, device="cpu")
    assert not cm.groups and set(cm.states) == {"run0.conv", "run0.scan"}
    s = cm.acquire_slot()
    cm.states["run0.scan"][s] += 1.0
    cm.release_slot(s)
    s2 = cm.acquire_slot()
    assert s2 == s and float(cm.states["run0.scan"][s2].abs().sum()) == 0.0     # a slot that is used again starts from zero
    sch = Scheduler(cm, max_batch=2, max_tokens_per_step=8)
    r = sch.add_request([1, 2, 3, 4, 5, 6, 7, 8, 9, 10], 12)
    plan = sch.schedule()
    assert [(x.start, x.count) for x in plan] == [(0, 8)]
    sch.complete(plan, [])
    plan = sch.schedule()
    assert [(x.start, x.count, x.samples) for x in plan] == [(8, 2, True)]


@pytest.mark.parametrize("which", ["mix", "plain", "one"])
def test_plain_implementation_is_causal(which):
    """The logits of a prefix do not change when tokens follow (what lets the engine cut a prompt anywhere)."""
    cfg = rh.config(which)
    W = rh.make_weights(cfg, 1)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(2)).tolist()
    full, _ = plain.forward(cfg, W, toks)
    part, _ = plain.forward(cfg, W, toks[:17])
    assert torch.allclose(full[:17], part, atol=1e-9, rtol=0)


def test_plain_window_and_sink():
    """One query, keys with known scores: the window cuts at exactly ``size`` keys, the sink takes its share."""
    T = 6
    vis = plain.causal_mask(T, window=3)
    assert vis[5].tolist() == [False, False, False, True, True, True] and vis[1].tolist() == [True, True, False, False, False, False]
    scores = torch.zeros(T, T, dtype=torch.float64)
    p = plain.softmax_rows(scores, vis, sink=torch.tensor(0.0, dtype=torch.float64))
    assert abs(float(p[5].sum()) - 0.75) < 1e-12 and abs(float(p[0].sum()) - 0.5) < 1e-12


def test_config_round_trip_through_a_folder(tmp_path):
    from delta_b200.config.registry import read_config
    cfg = rh.config("mix")
    folder = rh.write_folder(tmp_path, "m", cfg, rh.make_weights(cfg, 0))
    arch, typed = read_config(folder)
    assert arch.name == "Roletar" and typed.streams == 3 and typed.layers[1].mixer["mask"]["size"] == 21
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Roletar"
