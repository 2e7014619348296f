"""The Pibalorn design in the engine against the plain float64 implementation, on the GPU, in 32 bit and in bfloat16:
each mechanism alone (one-mechanism models, single kernels, and the stream after every layer run), each request whole,
prefill against token-by-token decoding, portions down to two tokens, mixed batches with pages, slots and states that
are used again, far keys across many tiny pages, long decoding, and greedy generation through ``LMBackend``, the
command line and the replay command."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import helpers
import pibalorn_helpers as ph
import plain_pibalorn as plain

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
# 32 bit: the largest difference of a logit (or a stream entry) as a fraction of the largest value of its request's
# reference.  bfloat16: the root mean square of a position's differences as a fraction of that of the request's
# reference logits, and at most three times what rounding alone causes.
TOL = {"float32": 2e-5, "bfloat16": 6e-2}
LENGTHS = {"wide": [250, 5, 199, 64], "mix": [3, 37, 60, 121], "odd": [1, 7, 26, 45], "one": [2, 25, 33, 58], "sharp": [1, 40, 97, 150], "only_attention": [2, 30, 47],
           "only_lightning": [1, 9, 40, 75], "only_experts": [1, 6, 21, 50], "only_pairs": [1, 2, 19], "pairs_many": [2, 33]}
_cache = {}


def model(tmp_path_factory, which):
    if which not in _cache:
        cfg = ph.config(which)
        W = ph.make_weights(cfg, 17 + len(which))
        folder = ph.write_folder(tmp_path_factory.mktemp("pibalorn"), which, cfg, W)
        _cache[which] = (cfg, W, folder)
    return _cache[which]


def make_runner(folder, which, dtype, num_pages=None, max_batch=4, max_seq_len=256, **kw):
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner
    ps = ph.PAGE_SIZE[which]
    cfg = EngineConfig(max_batch=max_batch, max_seq_len=max_seq_len, page_size=ps, dtype=dtype,
                       num_pages=num_pages if num_pages is not None else max_batch * (max_seq_len // ps), **kw)
    return ModelRunner(folder, engine_config=cfg)


def rounding_noise(cfg, W, toks, refs):
    out = []
    for t, ref in zip(toks, refs):
        with plain.rounding("bfloat16"):
            em = plain.forward(cfg, W, t)[0]
        out.append((em - ref).pow(2).mean(dim=1).sqrt().max().item())
    return out


def compare(results, refs, lengths, dtype, what, noise=None):
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
        allowed = TOL[dtype] * scale
        if noise is not None:      # a router's close call that flips under bfloat16 rounding is rounding noise too
            allowed = max(allowed, 3.0 * noise[i % len(noise)])
        bad = (err > allowed).nonzero()
        if bad.numel():
            p = int(bad[0, 0])
            raise AssertionError(f"{what}: request {i} first differs at position {p} (of {n}): error {err[p].item():.3e}, "
                                 f"allowed {allowed:.3e}")
        worst = max(worst, err.max().item() / scale)
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(LENGTHS))
def test_every_way_of_cutting(tmp_path_factory, which, dtype):
    cfg, W, folder = model(tmp_path_factory, which)
    lengths = LENGTHS[which]
    toks = [helpers.random_tokens(n, cfg["vocab"], 200 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    ps = ph.PAGE_SIZE[which]
    runner = make_runner(folder, which, dtype)
    noise = rounding_noise(cfg, W, toks, refs) if dtype == "bfloat16" else None
    worst = {}
    worst["whole"] = compare(helpers.run_schedule(runner, toks, helpers.whole(lengths)), refs, lengths, dtype, "whole", noise)
    worst["one by one"] = compare(helpers.run_schedule(runner, toks, helpers.last_one_by_one(lengths)), refs, lengths, dtype,
                                  "last 32 one by one", noise)
    for seed, sizes in ((1, (7, 2, 13, 2, 5, 3, 16, 2, 9)), (2, (2, 2, 3, 31, 2, 17, 33, 40))):
        res = helpers.run_schedule(runner, toks, helpers.changing_portions(lengths, seed=seed, sizes=sizes))
        worst[f"portions {seed}"] = compare(res, refs, lengths, dtype, "changing portions", noise)
    # mixed: more requests than slots, and a pool so small that pages of finished requests are used again
    prompt_lens = [max(1, n // 2) for n in lengths]
    steps, ends = helpers.mixed(lengths * 3, prompt_lens * 3, seed=3, max_live=3)
    tight = make_runner(folder, which, dtype, num_pages=helpers.peak_pages(steps, ends, ps), max_batch=3)
    res = helpers.run_schedule(tight, toks * 3, steps, ends)
    worst["mixed"] = compare(res, refs * 3, lengths * 3, dtype, "mixed with pages, slots and states used again", noise)
    print(f"\nworst logit error {which} {dtype}: " + ", ".join(f"{k} {v:.2e}" for k, v in worst.items()))


@pytest.mark.parametrize("which", ["mix", "odd", "one", "only_attention", "only_lightning", "only_experts", "only_pairs"])
def test_stream_after_every_layer_run(tmp_path_factory, which):
    """32 bit: the residual stream after every run of a layer, for a prompt in one step and for the same prompt cut in two."""
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


@pytest.mark.parametrize("which,dtype", [("mix", "float32"), ("odd", "float32"), ("mix", "bfloat16")])
def test_long_decoding(tmp_path_factory, which, dtype):
    """A short prompt, then 180 tokens one by one: pages fill one after the other, the recurrent state and the previous token
    are carried 180 times."""
    cfg, W, folder = model(tmp_path_factory, which)
    n = 185
    toks = [helpers.random_tokens(n, cfg["vocab"], 9)]
    refs = [plain.forward(cfg, W, toks[0])[0]]
    runner = make_runner(folder, which, dtype, max_batch=1)
    steps = [[(0, 0, 5)]] + [[(0, p, 1)] for p in range(5, n)]
    res = helpers.run_schedule(runner, toks, steps)
    print("\nlong decoding worst", compare(res, refs, [n], dtype, "long decoding"))
    assert all(g.pool.held_pages == 0 for g in runner.cache.groups.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["only_lightning", "mix", "odd"])
def test_long_portions_run_their_chunks_in_parallel(tmp_path_factory, which, dtype):
    """Portions long enough for the chunk-parallel recurrence: several chunks, one that ends in the middle of a chunk, rows of
    unequal length in one batch (some a single token), and a state carried on into single tokens afterwards."""
    cfg, W, folder = model(tmp_path_factory, which)
    lengths = [150, 9, 117, 33]
    toks = [helpers.random_tokens(n, cfg["vocab"], 300 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    runner = make_runner(folder, which, dtype)
    steps = [[(0, 0, 100), (1, 0, 8), (2, 0, 17)], [(0, 100, 41), (1, 8, 1), (2, 17, 97), (3, 0, 32)], [(0, 141, 1), (3, 32, 1), (2, 114, 3)]]
    steps += [[(0, p, 1)] for p in range(142, 150)]
    res = helpers.run_schedule(runner, toks, steps)
    noise = rounding_noise(cfg, W, toks, refs) if dtype == "bfloat16" else None
    print("\nchunks in parallel worst", compare(res, refs, lengths, dtype, "long portions", noise))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_at_the_edges_of_chunks(tmp_path_factory, dtype):
    """Portions of exactly one and two chunks, one token more and one less, on both sides of the length from which the chunks run
    in parallel; every request goes on with a portion that starts in the middle of a chunk and ends on a chunk's edge."""
    from delta_b200.kernels import ops
    from delta_b200.parts import decay_attention
    c = ops.decay_attention_chunk()
    assert decay_attention.PARALLEL_FROM == 2 * c + 1
    cfg, W, folder = model(tmp_path_factory, "only_lightning")
    first = [c, c + 1, 2 * c, 2 * c + 1, 3 * c - 1, 1]
    lengths = [n + (4 * c - n) for n in first]           # every request ends at 4 chunks
    toks = [helpers.random_tokens(n, cfg["vocab"], 500 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    noise = rounding_noise(cfg, W, toks, refs) if dtype == "bfloat16" else None
    for together in (True, False):      # the rows in one batch (the longest decides the path), and each alone (its own path)
        runner = make_runner(folder, "only_lightning", dtype, max_batch=len(first))
        if together:
            steps = [[(i, 0, n) for i, n in enumerate(first)], [(i, n, lengths[i] - n) for i, n in enumerate(first)]]
        else:
            steps = [[(i, 0, n)] for i, n in enumerate(first)] + [[(i, n, lengths[i] - n)] for i, n in enumerate(first)]
        res = helpers.run_schedule(runner, toks, steps)
        compare(res, refs, lengths, dtype, f"chunk edges, together={together}", noise)


def test_a_slot_used_again_starts_clean(tmp_path_factory):
    """Request B after request A in the same slot and pages equals B alone: state, previous token and cache of A are gone."""
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_carries_the_weight(tmp_path_factory, dtype):
    """Weights made so that one score stands out: the key matrix is a permutation P and token B's embedding is P times token
    A's, so the query of B (late in the prompt) meets the key of A (near its start, in the first page of many small ones) with
    the largest score there is, and no other key comes close.  A kernel that misses that key, in a prompt portion or in a
    single decoded token, changes the logits at B beyond any tolerance."""
    d = 16
    cfg = dict(architecture="Pibalorn", norm=dict(eps=1e-5), vocab=64, width=d, layers=[ph.bare(ph.attention(1, 1, d, 3.0))])
    g = torch.Generator().manual_seed(77)
    W = ph.make_weights(cfg, 9)
    perm = torch.randperm(d, generator=g)
    P = torch.eye(d)[perm]
    W["embed"][1] = P @ W["embed"][0]
    W["l0.mix.q"], W["l0.mix.k"], W["l0.mix.o"] = torch.eye(d), P.clone(), torch.eye(d) * 0.5
    W["l0.norm1"] = torch.ones(d)
    folder = ph.write_folder(tmp_path_factory.mktemp("far"), "far", cfg, W)
    n, a_at, b_at = 150, 3, 140
    toks = [2 + t % 62 for t in helpers.random_tokens(n, 62, 8)]
    toks[a_at], toks[b_at] = 0, 1
    ref = plain.forward(cfg, W, toks)[0]
    without = list(toks)
    without[a_at] = 5
    changed = (plain.forward(cfg, W, without)[0][b_at] - ref[b_at]).abs().max().item()
    assert changed > 0.2 * ref[b_at].abs().max().item(), "the crafted key does not carry the weight"
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner
    runner = ModelRunner(folder, engine_config=EngineConfig(max_batch=2, max_seq_len=160, page_size=4, dtype=dtype, num_pages=80))
    noise = rounding_noise(cfg, W, [toks], [ref]) if dtype == "bfloat16" else None
    for what, steps in (("whole", [[(0, 0, n)]]), ("B decoded alone", [[(0, 0, b_at)]] + [[(0, p, 1)] for p in range(b_at, n)]),
                        ("B opens a portion", [[(0, 0, 2)], [(0, 2, b_at - 2)], [(0, b_at, n - b_at)]]),
                        ("B ends a portion", [[(0, 0, a_at)], [(0, a_at, 1)], [(0, a_at + 1, b_at - a_at)], [(0, b_at + 1, n - b_at - 1)]])):
        compare(helpers.run_schedule(runner, [toks], steps), [ref], [n], dtype, what, noise)


# ---- single kernels against their equations --------------------------------------------------------------------

def _rows(lens, slots, dev):
    i32 = torch.int32
    starts = [sum(lens[:i]) for i in range(len(lens))]
    return dict(row_slot=torch.tensor(slots, dtype=i32, device=dev), row_q_start=torch.tensor(starts, dtype=i32, device=dev),
                row_q_len=torch.tensor(lens, dtype=i32, device=dev))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv", [(2, 16, 8), (3, 6, 10), (1, 128, 128), (2, 64, 200)])
def test_decay_attention_kernel(H, dk, dv, dtype):
    """Rows of unequal length, one of them several chunks long and one a single token, from states that are not zero; a decay
    so small that its powers underflow and one close to 1."""
    from delta_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(H * 100 + dk)
    lens, slots = [70, 1, 33, 2], [2, 0, 3, 1]
    T = sum(lens)
    n = 2 * H * dk + H * dv
    src = (torch.randn(T, n + 5, generator=g) * 0.8).to(dtype)
    decays = [0.999, 0.02, 0.7][:H]
    state0 = torch.randn(5, H, dk, dv, generator=g) * 0.3
    state = state0.clone().to(dev)
    out = torch.empty(T, H * dv, dtype=torch.float32, device=dev)
    ops.decay_attention(src.to(dev), 0, H * dk, 2 * H * dk, torch.tensor(decays, dtype=torch.float64, device=dev), state, out, H=H, dk=dk,
                        dv=dv, **_rows(lens, slots, dev))
    x = torch.nn.functional.silu(src.double())
    t0 = 0
    worst = 0.0
    for L, s in zip(lens, slots):
        for h in range(H):
            S = state0[s, h].double().clone()
            for t in range(t0, t0 + L):
                q, k = x[t, h * dk:(h + 1) * dk], x[t, H * dk + h * dk:H * dk + (h + 1) * dk]
                v = x[t, 2 * H * dk + h * dv:2 * H * dk + (h + 1) * dv]
                S = decays[h] * S + torch.outer(k, v)
                o = S.T @ q
                worst = max(worst, ((out[t, h * dv:(h + 1) * dv].cpu().double() - o).abs().max() / (o.abs().max() + 1e-3)).item())
            worst = max(worst, ((state[s, h].cpu().double() - S).abs().max() / (S.abs().max() + 1e-3)).item())
        t0 += L
    assert torch.equal(state[4].cpu(), state0[4])       # a slot no row names is left alone
    assert worst < 2e-5, worst
    # the same rows with their chunks in parallel: outputs and end states agree with the path that takes the chunks in turn
    if ops.decay_attention_chunked_supported(dk, dv):
        chunk = ops.decay_attention_chunk()
        counts = [-(-n // chunk) for n in lens]
        base = torch.tensor([sum(counts[:i]) for i in range(len(lens))], dtype=torch.int32, device=dev)
        work = torch.empty(sum(counts) * H * dk * dv, dtype=torch.float32, device=dev)
        state2 = state0.clone().to(dev)
        out2 = torch.empty_like(out)
        ops.decay_attention_chunked(src.to(dev), 0, H * dk, 2 * H * dk, torch.tensor(decays, dtype=torch.float64, device=dev), state2, out2,
                                    work, base, max(counts), H=H, dk=dk, dv=dv, **_rows(lens, slots, dev))
        scale = out.abs().max().item()
        assert (out2 - out).abs().max().item() < 2e-5 * scale
        assert (state2 - state).abs().max().item() < 2e-5 * state.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,F,d", [(1, 4, 2, 12, 40), (37, 7, 3, 24, 40), (130, 5, 5, 9, 50), (64, 3, 1, 70, 33)])
def test_experts_kernels(T, E, top, F, d, dtype):
    """Routing, sorting into tiles, both products and the weighted sum against a loop over tokens; all tokens to one expert
    (a logit column far above the others) fills several tiles of that expert and none of the others."""
    from delta_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(T + E)
    for crowd in (False, True):
        x = torch.randn(T, d, generator=g).to(dtype)
        w1 = (torch.randn(E, 2 * F, d, generator=g) / d ** 0.5).to(dtype)
        w2 = (torch.randn(E, d, F, generator=g) / F ** 0.5).to(dtype)
        z = torch.randn(T, E + 1, generator=g)
        if crowd:
            z[:, E - 1] += 50.0
        choice = torch.empty(T, top, dtype=torch.int32, device=dev)
        weight = torch.empty(T, top, dtype=torch.float32, device=dev)
        ops.router_topk(z.to(dev), E, top, choice, weight)
        vals, idx = torch.topk(z[:, :E], top, dim=-1)
        assert torch.equal(choice.cpu().long(), idx)
        assert torch.allclose(weight.cpu(), torch.softmax(vals, -1), atol=1e-6)
        tile = ops.experts_tile_rows()
        cap = -(-(T * top + (tile - 1) * min(E, T * top)) // tile) * tile
        sorted_slots = torch.empty(cap, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(cap // tile, dtype=torch.int32, device=dev)
        ops.experts_align(choice, E, sorted_slots, tile_expert)
        ss, te = sorted_slots.cpu(), tile_expert.cpu()
        assert sorted(int(s) for s in ss if s >= 0) == list(range(T * top))
        for p, s in enumerate(ss.tolist()):
            if s >= 0:
                assert int(te[p // tile]) == int(choice.view(-1)[s])
        y = torch.empty(cap, F, dtype=dtype, device=dev)
        ops.experts_gemm(x.to(dev), w1.to(dev), y, sorted_slots, tile_expert, top=top, n=F, k=d, act=True, limit=0.9)
        zs = torch.empty(T * top, d, dtype=torch.float32, device=dev)
        ops.experts_gemm(y, w2.to(dev), zs, sorted_slots, tile_expert, top=top, n=d, k=F)
        shared = torch.randn(T, d, generator=g).to(dtype)
        out = torch.empty(T, d, dtype=dtype, device=dev)
        zd = z.to(dev)
        ops.experts_combine(zs, weight, out, shared=shared.to(dev), gate_logit=zd.data_ptr() + E * 4, gate_stride=E + 1)
        ref = torch.zeros(T, d, dtype=torch.float64)
        rnd = (lambda a: a.to(dtype).double())
        for t in range(T):
            for j in range(top):
                e = int(idx[t, j])
                gu = rnd(x[t].double() @ w1[e].double().T)
                gg, uu = gu[:F].clamp(max=0.9), gu[F:].clamp(-0.9, 0.9)
                yy = rnd(gg * torch.sigmoid(1.702 * gg) * (uu + 1))
                ref[t] += torch.softmax(vals[t].double(), -1)[j] * (yy @ w2[e].double().T)
            ref[t] += torch.sigmoid(z[t, E].double()) * shared[t].double()
        err = (out.cpu().double() - ref).abs().max().item() / ref.abs().max().item()
        assert err < (2e-5 if dtype == torch.float32 else 2e-2), (crowd, err)


@pytest.mark.parametrize("T,E,top,F,d", [(700, 4, 2, 64, 128), (300, 3, 3, 128, 72), (1030, 5, 1, 192, 256)])
def test_experts_products_on_tcgen05(T, E, top, F, d):
    """The experts' products through the tcgen05 kernel (tiles of 128 rows gathered side by side) against the warp-level MMA
    path on the same routing: an expert with no rows at all, one with more than two tiles, and a tile that is nearly empty."""
    from delta_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(T + F)
    bf = torch.bfloat16
    x = torch.randn(T, d, generator=g).to(bf).to(dev)
    w1 = (torch.randn(E, 2 * F, d, generator=g) / d ** 0.5).to(bf).to(dev)
    w2 = (torch.randn(E, d, F, generator=g) / F ** 0.5).to(bf).to(dev)
    z = torch.randn(T, E, generator=g)
    if E > top:
        z[:, 1] -= 100.0             # nobody chooses expert 1
    choice = torch.empty(T, top, dtype=torch.int32, device=dev)
    weight = torch.empty(T, top, dtype=torch.float32, device=dev)
    ops.router_topk(z.to(dev), E, top, choice, weight)
    assert ops.experts_gemm_tc_supported(F, d, True) and ops.experts_gemm_tc_supported(d, F, False)
    outs = []
    err = ops.new_error_record(dev)
    for tile in (ops.experts_tile_rows(), 128):
        cap = -(-(T * top + (tile - 1) * min(E, T * top)) // tile) * tile
        ss = torch.empty(cap, dtype=torch.int32, device=dev)
        te = torch.empty(cap // tile, dtype=torch.int32, device=dev)
        ops.experts_align(choice, E, ss, te, tile)
        y = torch.zeros(cap, F, dtype=bf, device=dev)
        zs = torch.full((T * top, d), float("nan"), dtype=torch.float32, device=dev)
        if tile == 128:
            rows = ops.experts_gather(x, ss, top, torch.empty(cap, d, dtype=bf, device=dev))
            ops.experts_gemm_tc(rows, w1, y, te, tile, n=F, glu=True, limit=0.9, err=err)
            ops.experts_gemm_tc(y, w2, zs, te, tile, n=d, row_map=ss, err=err)
            ops.raise_if_error(err)
        else:
            ops.experts_gemm(x, w1, y, ss, te, top=top, n=F, k=d, act=True, limit=0.9)
            ops.experts_gemm(y, w2, zs, ss, te, top=top, n=d, k=F)
        outs.append(zs.cpu())
    assert torch.isfinite(outs[1]).all()
    assert (outs[0] - outs[1]).abs().max().item() <= 2e-2 * outs[0].abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,d,extra", [(1, 4, 2, 40, 1), (19, 7, 7, 50, 0), (70, 33, 5, 333, 1), (9, 3, 1, 2048, 1)])
def test_router_kernel(T, E, top, d, extra, dtype):
    """The router's product in 32 bit with its choice: logits, the chosen experts in the order of their logits, the softmax over
    the chosen ones; a further row of the matrix (a gate's) is computed and left out of the choice."""
    from delta_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(T * 7 + E)
    x = torch.randn(T, d, generator=g).to(dtype)
    w = (torch.randn(E + extra, d, generator=g) * 3 / d ** 0.5).to(dtype)
    if extra:
        w[E] = w[:E].abs().sum(0)          # a row whose logit is far above every expert's
    z = torch.empty(T, E + extra, dtype=torch.float32, device=dev)
    choice = torch.empty(T, top, dtype=torch.int32, device=dev)
    weight = torch.empty(T, top, dtype=torch.float32, device=dev)
    ops.router(x.to(dev), w.to(dev), E, top, z, choice, weight)
    ref = x.double() @ w.double().T
    assert (z.cpu().double() - ref).abs().max().item() < 1e-5 * max(1.0, ref.abs().max().item())
    vals, idx = torch.topk(z.cpu()[:, :E], top, dim=-1)
    assert torch.equal(choice.cpu().long(), idx)
    assert torch.allclose(weight.cpu(), torch.softmax(vals, -1), atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("F", [24, 9, 256])
@pytest.mark.parametrize("limit", [-1.0, 0.0, 1.2])
def test_glu_clamped_kernel(F, limit, dtype):
    """Both forms of the kernel (eight entries a thread, one entry a thread); no limit, a limit of zero taken literally, a limit."""
    from delta_b200.kernels import ops
    g = torch.Generator().manual_seed(F)
    gu = (torch.randn(13, 2 * F, generator=g) * 2).to(dtype)
    out = torch.empty(13, F, dtype=dtype, device="cuda:0")
    ops.glu_clamped(gu.to("cuda:0"), out, limit)
    a, b = gu[:, :F].double(), gu[:, F:].double()
    if limit >= 0:
        a, b = a.clamp(max=limit), b.clamp(-limit, limit)
    ref = a * torch.sigmoid(1.702 * a) * (b + 1)
    assert (out.cpu().double() - ref).abs().max().item() <= (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["layer", "rms"])
def test_residual_norm_kernel(kind, dtype):
    from delta_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(3)
    T, d = 9, 50
    X = torch.randn(T, d, generator=g) * 3 + 5.0          # a mean far from zero: the variance is taken about the mean
    y1, y2 = torch.randn(T, d, generator=g).to(dtype), torch.randn(T, d, generator=g).to(dtype)
    e, vec, w = torch.randn(T, d, generator=g), torch.randn(d, generator=g), torch.rand(d, generator=g) + 0.5
    rows = torch.tensor([7, 2, 2], dtype=torch.int32)
    Xd = X.clone().to(dev)
    out = torch.empty(3, d, dtype=dtype, device=dev)
    ops.residual_norm(Xd, out, updates=(y1.to(dev), y2.to(dev)), extra=e.to(dev), vec=vec.to(dev), weight=w.to(dev), eps=1e-5, kind=kind,
                      rows=rows.to(dev), write_back=False)
    assert torch.equal(Xd.cpu(), X)
    s = X.double() + (y1.double() + y2.double()) + e.double() + vec.double()
    ref = (plain.layer_norm(s, w, 1e-5) if kind == "layer" else plain.unit_rms(s, 1e-5) * w.double())[rows.long()]
    assert (out.cpu().double() - ref).abs().max().item() < (1e-5 if dtype == torch.float32 else 3e-2)
    ops.residual_norm(Xd, None, updates=(y1.to(dev),))
    assert (Xd.cpu().double() - (X.double() + y1.double())).abs().max().item() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rows_append_unit_kernel(dtype):
    """Queries and keys rotated in halves on a leading part, then unit-normed; the value is the key as it came."""
    from delta_b200.kernels import ops
    from delta_b200.parts.rope import RotaryPositions
    dev = "cuda:0"
    g = torch.Generator().manual_seed(4)
    H, KV, dk, ps, rot = 3, 2, 10, 4, 6
    pos = torch.tensor([0, 5, 6, 11], dtype=torch.int32)
    T = len(pos)
    src = torch.randn(T, (H + KV) * dk + 3, generator=g).to(dtype)
    cache = torch.zeros(5, KV, ps, 2 * dk, dtype=dtype, device=dev)
    bt = torch.tensor([[3, 1, 4]], dtype=torch.int32, device=dev)
    table = RotaryPositions(rot, 100.0, 16, interleaved=False).table(dev)
    sd = src.clone().to(dev)
    ops.rows_append_unit(sd, pos.to(dev), torch.zeros(T, dtype=torch.int32, device=dev), bt, cache, H=H, KV=KV, dk=dk, dv=dk, ps=ps,
                         row_width=2 * dk, k_off=0, v_off=dk, table=table, rot_dims=rot, interleaved=False, unit_eps=1e-5,
                         value_from_key=True)
    heads = src[:, :(H + KV) * dk].double().view(T, H + KV, dk)
    want = plain.unit_rms(plain.rotate_half(heads, pos, 100.0, rot), 1e-5)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert (sd.cpu()[:, :H * dk].double().view(T, H, dk) - want[:, :H]).abs().max().item() < tol
    for t, p in enumerate(pos.tolist()):
        page = int(bt[0, p // ps])
        row = cache[page, :, p % ps].cpu().double()
        assert (row[:, :dk] - want[t, H:]).abs().max().item() < tol
        assert torch.equal(row[:, dk:], heads[t, H:])
    assert torch.equal(sd.cpu()[:, H * dk:], src[:, H * dk:])      # keys are not changed in place


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv", [(2, 16, 8), (3, 6, 12), (1, 128, 128), (2, 50, 200)])
def test_decay_attention_step_kernel(H, dk, dv, dtype):
    """Steps of single tokens: the kernel that streams the state once agrees with the chunked one, outputs and states, for rows
    in slots out of order and from states that are not zero."""
    from delta_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(dk + dv)
    slots = [3, 0, 2]
    rows = len(slots)
    src = (torch.randn(rows, 2 * H * dk + H * dv + 3, generator=g) * 0.8).to(dtype).to(dev)
    decays = torch.tensor([0.999, 0.3, 0.9][:H], dtype=torch.float64, device=dev)
    state0 = torch.randn(5, H, dk, dv, generator=g) * 0.5
    assert ops.decay_attention_step_supported(dk, dv)
    outs, states = [], []
    for step in (False, True):
        state = state0.clone().to(dev)
        out = torch.empty(rows, H * dv, dtype=torch.float32, device=dev)
        kw = dict(H=H, dk=dk, dv=dv)
        r = _rows([1] * rows, slots, dev)
        if step:
            ops.decay_attention_step(src, 0, H * dk, 2 * H * dk, decays, state, out, row_slot=r["row_slot"], row_q_start=r["row_q_start"], **kw)
        else:
            ops.decay_attention(src, 0, H * dk, 2 * H * dk, decays, state, out, **r, **kw)
        outs.append(out.cpu())
        states.append(state.cpu())
    assert (outs[0] - outs[1]).abs().max().item() <= 1e-5 * outs[0].abs().max().item()
    assert (states[0] - states[1]).abs().max().item() <= 1e-5 * states[0].abs().max().item()
    assert torch.equal(states[1][1], state0[1]) and torch.equal(states[1][4], state0[4])


# ---- through the engine's own entry points -----------------------------------------------------------------------

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


def test_generation_survives_preemption(tmp_path_factory):
    """A pool too small for all running requests: the youngest is preempted and computed again from a fresh slot, whose
    state and previous token start over; the tokens are those of the plain implementation all the same."""
    from delta_b200.engine import LMBackend
    cfg, W, folder = model(tmp_path_factory, "mix")
    prompts = [helpers.random_tokens(n, cfg["vocab"], 80 + n) for n in (14, 15, 13)]
    want = [greedy_plain(cfg, W, p, 12) for p in prompts]
    e = LMBackend(dtype="float32", device="cuda:0")
    e.load_model(str(folder))
    e.setup_caches(max_batch_size=3, max_seq_length=32, page_size=4, max_tokens_per_step=16, num_pages=15)
    assert e.generate(prompts, 12) == want
    assert e.scheduler.stats["preemptions"] >= 1


def test_trace_replay_command(tmp_path_factory, tmp_path):
    """``bin/trace_run`` on a Pibalorn folder: a prompt in portions beside another request's single tokens."""
    cfg, W, folder = model(tmp_path_factory, "odd")
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
    """``python -m delta_b200.cli`` on a Pibalorn folder: the model class comes from config.json, prompts are scheduled and sampled."""
    import random
    from delta_b200 import cli
    cfg, W, folder = model(tmp_path_factory, "one")
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
