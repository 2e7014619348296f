"""The Roletar design in the engine against the plain float64 implementation, on the GPU, in 32 bit and in
bfloat16: each mechanism alone (one-layer models, and the stream after every layer run), each request whole,
prefill against token-by-token decoding, portions down to two tokens, mixed batches with pages, slots and states
that are used again, long decoding across windows and pages, and greedy generation through ``LMBackend``."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import helpers
import plain_roletar as plain
import roletar_helpers as rh

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
# 32 bit differs from float64 by the rounding of sums: the largest difference allowed to a logit (or a stream entry) is this
# fraction of the largest value of its request's reference.  bfloat16 differs by the rounding of activations between
# products, which single logits of a small model feel unevenly: there the root mean square of a position's differences is
# bounded, as a fraction of the root mean square of the request's reference logits.
TOL = {"float32": 2e-5, "bfloat16": 5e-2}
LENGTHS = {"odd": [1, 7, 26, 45], "mix": [3, 37, 60, 121], "plain": [1, 19, 44, 70], "one": [2, 25, 33, 58], "only_mamba": [1, 9, 40],
           "only_attention": [2, 30, 47], "only_latent": [2, 30, 47], "only_mlp_streams": [1, 6, 21]}
_cache = {}


def model(tmp_path_factory, which):
    if which not in _cache:
        cfg = rh.config(which)
        W = rh.make_weights(cfg, 11 + len(which))
        folder = rh.write_folder(tmp_path_factory.mktemp("roletar"), which, cfg, W)
        _cache[which] = (cfg, W, folder)
    return _cache[which]


def make_runner(folder, which, dtype, num_pages=None, max_batch=4, max_seq_len=256, **kw):
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner
    ps = rh.PAGE_SIZE[which]
    cfg = EngineConfig(max_batch=max_batch, max_seq_len=max_seq_len, page_size=ps, dtype=dtype,
                       num_pages=num_pages if num_pages is not None else max_batch * (max_seq_len // ps), **kw)
    return ModelRunner(folder, engine_config=cfg)


def rounding_noise(cfg, W, toks, refs):
    """Per request, the largest root-mean-square difference of a position's logits between the plain implementation that
    rounds every product and activation to bfloat16 once and the one that rounds nothing: what rounding alone causes."""
    out = []
    for t, ref in zip(toks, refs):
        with plain.rounding("bfloat16"):
            em = plain.forward(cfg, W, t)[0]
        out.append((em - ref).pow(2).mean(dim=1).sqrt().max().item())
    return out


def compare(results, refs, lengths, dtype, what, noise=None):
    """``noise`` (bfloat16): a position may differ by three times what rounding alone causes in its request, and no more."""
    worst = 0.0
    for i, n in enumerate(lengths):
        got = helpers.stack_positions(results, i, n).double()
        if dtype == "float32":
            err = (got - refs[i]).abs().max(dim=1).values
            scale = refs[i].abs().max().item()
        else:
            err = (got - refs[i]).pow(2).mean(dim=1).sqrt()
            scale = refs[i].pow(2).mean().sqrt().item()
            if noise is not None:
                over = (err > 3.0 * noise[i % len(noise)] + 1e-6).nonzero()
                assert not over.numel(), (f"{what}: request {i} position {int(over[0, 0])}: error {err[int(over[0, 0])].item():.3e} is more than "
                                          f"three times the rounding noise {noise[i % len(noise)]:.3e}")
        bad = (err > TOL[dtype] * scale).nonzero()
        if bad.numel():
            p = int(bad[0, 0])
            raise AssertionError(f"{what}: request {i} first differs at position {p} (of {n}): error {err[p].item():.3e}, "
                                 f"allowed {TOL[dtype] * scale:.3e}")
        worst = max(worst, err.max().item() / scale)
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["mix", "plain", "one", "odd", "only_mamba", "only_attention", "only_latent", "only_mlp_streams"])
def test_every_way_of_cutting(tmp_path_factory, which, dtype):
    cfg, W, folder = model(tmp_path_factory, which)
    lengths = LENGTHS[which]
    toks = [helpers.random_tokens(n, cfg["vocab"], 200 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    ps = rh.PAGE_SIZE[which]
    runner = make_runner(folder, which, dtype)
    noise = rounding_noise(cfg, W, toks, refs) if dtype == "bfloat16" else None
    worst = {}
    worst["whole"] = compare(helpers.run_schedule(runner, toks, helpers.whole(lengths)), refs, lengths, dtype, "whole", noise)
    worst["one by one"] = compare(helpers.run_schedule(runner, toks, helpers.last_one_by_one(lengths)), refs, lengths, dtype,
                                  "last 32 one by one", noise)
    for seed, sizes in ((1, (7, 2, 13, 2, 5, 3, 16, 2, 9)), (2, (2, 2, 3, 31, 2, 17))):
        res = helpers.run_schedule(runner, toks, helpers.changing_portions(lengths, seed=seed, sizes=sizes))
        worst[f"portions {seed}"] = compare(res, refs, lengths, dtype, "changing portions", noise)
    # mixed: more requests than slots, and a pool so small that pages of finished requests are used again
    prompt_lens = [max(1, n // 2) for n in lengths]
    steps, ends = helpers.mixed(lengths * 3, prompt_lens * 3, seed=3, max_live=3)
    tight = make_runner(folder, which, dtype, num_pages=helpers.peak_pages(steps, ends, ps), max_batch=3)
    res = helpers.run_schedule(tight, toks * 3, steps, ends)
    worst["mixed"] = compare(res, refs * 3, lengths * 3, dtype, "mixed with pages, slots and states used again", noise)
    print(f"\nworst logit error {which} {dtype}: " + ", ".join(f"{k} {v:.2e}" for k, v in worst.items()))


@pytest.mark.parametrize("which", ["mix", "plain", "one", "only_mamba", "only_attention", "only_latent", "only_mlp_streams"])
def test_stream_after_every_layer_run(tmp_path_factory, which):
    """32 bit: the summed stream copies after every run of a layer, for a prompt in one step and for the same
    prompt cut in two."""
    from delta_b200.engine.step import RowInput
    cfg, W, folder = model(tmp_path_factory, which)
    toks = helpers.random_tokens(29, cfg["vocab"], 5)
    _, after = plain.forward(cfg, W, toks)
    runner = make_runner(folder, which, "float32")
    for cut in (29, 11):
        slot = runner.cache.acquire_slot()
        got = []
        for a, b in ((0, cut), (cut, 29)):
            if a == b:
                continue
            runner.capture = {"layer_totals": []}
            runner.run_rows([RowInput(slot, toks[a:b], a, [])])
            got.append(torch.stack(runner.capture["layer_totals"]).cpu())
        runner.capture = None
        runner.cache.release_slot(slot)
        got = torch.cat(got, dim=1).double()
        assert got.shape == after.shape
        for r in range(after.shape[0]):
            err = (got[r] - after[r]).abs().max().item()
            assert err <= TOL["float32"] * after[r].abs().max().item(), f"{which}: layer run {r} differs by {err:.3e} (cut at {cut})"


@pytest.mark.parametrize("which,dtype", [("mix", "float32"), ("one", "float32"), ("mix", "bfloat16")])
def test_long_decoding(tmp_path_factory, which, dtype):
    """A short prompt, then 180 tokens one by one: windows pass over decoded tokens, pages fill and are given back,
    the recurrent state is carried 180 times."""
    cfg, W, folder = model(tmp_path_factory, which)
    n = 185
    toks = [helpers.random_tokens(n, cfg["vocab"], 9)]
    refs = [plain.forward(cfg, W, toks[0])[0]]
    runner = make_runner(folder, which, dtype, max_batch=1)
    steps = [[(0, 0, 5)]] + [[(0, p, 1)] for p in range(5, n)]
    res = helpers.run_schedule(runner, toks, steps)
    print("\nlong decoding worst", compare(res, refs, [n], dtype, "long decoding"))
    windowed = [g for g in runner.cache.groups.values() if g.spec.window]
    assert all(g.pool.held_pages == 0 for g in runner.cache.groups.values())
    assert windowed, "this test is meant for a model with a windowed layer"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["only_mamba", "mix", "one"])
def test_long_portions_run_in_segments(tmp_path_factory, monkeypatch, which, dtype):
    """Portions longer than a segment: the recurrence runs in parallel pieces that are stitched together.  With segments of
    16 tokens: portions of many segments, one that ends in the middle of a segment, rows of unequal length in one batch
    (some shorter than a segment), and a state that is carried on into single tokens afterwards."""
    from delta_b200.parts import selective_scan
    monkeypatch.setattr(selective_scan, "SEGMENT", 16)
    cfg, W, folder = model(tmp_path_factory, which)
    lengths = [150, 9, 77, 33]
    toks = [helpers.random_tokens(n, cfg["vocab"], 300 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    runner = make_runner(folder, which, dtype)
    steps = [[(0, 0, 100), (1, 0, 9), (2, 0, 17)], [(0, 100, 41), (2, 17, 60), (3, 0, 32)], [(0, 141, 1), (3, 32, 1)]]
    steps += [[(0, p, 1)] for p in range(142, 150)]
    res = helpers.run_schedule(runner, toks, steps)
    print("\nsegments worst", compare(res, refs, lengths, dtype, "portions in segments"))


def test_segments_of_the_real_length(tmp_path_factory):
    """The segment length the engine uses: one prompt of three and a half segments beside a short one."""
    from delta_b200.parts import selective_scan
    cfg, W, folder = model(tmp_path_factory, "only_mamba")
    n = 3 * selective_scan.SEGMENT + selective_scan.SEGMENT // 2 + 3
    lengths = [n, 20]
    toks = [helpers.random_tokens(m, cfg["vocab"], 400 + i) for i, m in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    runner = make_runner(folder, "only_mamba", "float32", max_seq_len=512)
    res = helpers.run_schedule(runner, toks, [[(0, 0, n - 2), (1, 0, 20)], [(0, n - 2, 2)]])
    compare(res, refs, lengths, "float32", "segments of the real length")


def test_a_slot_used_again_starts_clean(tmp_path_factory):
    """Request B after request A in the same slot and pages equals B alone (state and cache of A are gone)."""
    from delta_b200.engine.step import RowInput
    cfg, W, folder = model(tmp_path_factory, "mix")
    runner = make_runner(folder, "mix", "float32", max_batch=1, num_pages=8, max_seq_len=128)
    a, b = helpers.random_tokens(100, cfg["vocab"], 1), helpers.random_tokens(50, cfg["vocab"], 2)
    ref = plain.forward(cfg, W, b)[0]
    for toks in (a, b):
        slot = runner.cache.acquire_slot()
        assert slot == 0
        logits = runner.run_rows([RowInput(slot, toks, 0, list(range(len(toks))))])
        runner.cache.release_slot(slot)
    err = (logits.cpu().double() - ref).abs().max().item()
    assert err <= TOL["float32"] * ref.abs().max().item()


def greedy_plain(cfg, W, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        logits, _ = plain.forward(cfg, W, toks)
        toks.append(int(torch.argmax(logits[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("graph", [False, True])
def test_greedy_generation_through_the_backend(tmp_path_factory, graph):
    """``LMBackend``: more prompts than slots, a token budget that cuts prompts, decode steps (recorded or not)."""
    from delta_b200.engine import LMBackend
    cfg, W, folder = model(tmp_path_factory, "mix")
    prompts = [helpers.random_tokens(n, cfg["vocab"], 50 + n) for n in (4, 23, 9, 31, 2)]
    want = [greedy_plain(cfg, W, p, 10) for p in prompts]
    e = LMBackend(dtype="float32", device="cuda:0", cuda_graph_decode=graph)
    e.load_model(str(folder))
    e.setup_caches(max_batch_size=3, max_seq_length=64, page_size=16, max_tokens_per_step=16)
    got = e.generate(prompts, 10)
    assert got == want
    assert e.scheduler.stats["prefill_steps"] > 2
    if graph:
        assert e.runner.graph_replays > 0 and not e.runner.graph_fallbacks


def test_trace_replay_command(tmp_path_factory, tmp_path):
    """``bin/trace_run`` on a Roletar folder: a prompt in portions beside another request's single tokens."""
    cfg, W, folder = model(tmp_path_factory, "one")
    a, b = helpers.random_tokens(21, cfg["vocab"], 3), helpers.random_tokens(12, cfg["vocab"], 4)
    steps = [dict(step=0, entries=[dict(id="a", tokens=a[:7], want=[6])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=a[7:9], want=[0, 1]), dict(id="b", tokens=b[:11], want=[10])], end=[]),
             dict(step=2, entries=[dict(id="b", tokens=b[11:], want=[0]), dict(id="a", tokens=a[9:], want=[11])], end=["a", "b"])]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128", "--page-size", "4"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ra, rb = plain.forward(cfg, W, a)[0], plain.forward(cfg, W, b)[0]
    import numpy as np
    V = cfg["vocab"]
    got = {k: torch.from_numpy(np.fromfile(out / f"{k}.f32", dtype="<f4").reshape(-1, V)).double() for k in range(3)}
    want = {0: ra[[6]], 1: torch.cat([ra[[7, 8]], rb[[10]]]), 2: torch.cat([rb[[11]], ra[[20]]])}
    for k in range(3):
        assert got[k].shape == want[k].shape
        assert (got[k] - want[k]).abs().max().item() <= TOL["float32"] * want[k].abs().max().item()


def test_command_line_generates(tmp_path_factory, tmp_path):
    """``python -m delta_b200.cli`` on a Roletar folder: the model class comes from config.json, prompts are scheduled and sampled."""
    import random
    from delta_b200 import cli
    cfg, W, folder = model(tmp_path_factory, "plain")
    out = tmp_path / "result.json"
    rc = cli.main(["--model", str(folder), "--B", "3", "--max_len", "128", "--dataset", "random", "--prompt_len", "19", "--num_samples", "5",
                   "--max_new_tokens", "6", "--dtype", "float32", "--max_tokens_per_step", "32", "--out", str(out)])
    assert rc == 0
    res = json.loads(out.read_text())
    assert res["summary"]["requests"] == 5 and res["summary"]["generated_tokens"] == 30
    rng = random.Random(123)       # the command line's default seed draws the prompts
    prompt = [rng.randrange(cfg["vocab"]) for _ in range(19)]
    first = [r for r in res["results"] if r["request_id"] == 0][0]
    assert first["output_ids"] == greedy_plain(cfg, W, prompt, 6)
