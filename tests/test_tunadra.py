"""Tunadra: every mechanism alone against the plain implementation, then whole models in every
cutting of the work (whole prompts, token by token, portions down to two tokens, unequal requests in
one batch, pages and state slots given back and used again), long decoding from captured steps, the
trace tool and greedy generation through the engine."""

from __future__ import annotations

import json
import subprocess
import sys

import numpy as np
import pytest
import torch

from gunedra_helpers import MEAN_TOLERANCE, TOLERANCE, Replay, as_float64, row_error, write_folder
from helpers import TRACE_RUN
from plain import tunadra_plain as plain
from test_parts import context_for
from tunadra_helpers import ALPHA, CONFIGS, attention_layer, draw_weights, moe, wkv_layer

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CLOSE = {"float32": dict(atol=2e-5, rtol=2e-5), "bfloat16": dict(atol=5e-2, rtol=3e-2)}


def rounded(array: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(array)).to(dtype)


def on_device(array: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32)).cuda()


# --- kernels and parts alone ---------------------------------------------------------------------------


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,streams", [(48, 3), (40, 1), (4100, 2)])
def test_sinusoid_embedding_fills_every_stream(name, hidden, streams):
    """Positions from a request's start to tens of thousands: the angle is position times a tabulated
    frequency in 32-bit, so the bound grows with the position."""
    from llm_inference_b200.parts import PartSpec, build_part

    dtype, vocab = DTYPES[name], 37
    starts, runs = [0, 977, 40000], [5, 3, 2]
    _, _, ctx = context_for({}, dtype, runs)
    ctx.positions.copy_(torch.cat([torch.arange(s, s + r, dtype=torch.int32) for s, r in zip(starts, runs)]).cuda())
    rng = np.random.default_rng(hidden)
    part = build_part("embedding", PartSpec("sinusoid_embedding", dict(name="e", vocab_size=vocab, hidden_size=hidden, scale=2.5, streams=streams)))
    table = rounded(rng.normal(0, 1, (vocab, hidden)), torch.bfloat16)
    part.load({"e": table}, dtype, ctx.device)
    ids = rng.integers(0, vocab, sum(runs))
    ctx.token_ids.copy_(torch.from_numpy(ids.astype(np.int32)).cuda())
    x = part.forward(ctx).cpu().numpy().reshape(sum(runs), streams, hidden)
    positions = np.concatenate([np.arange(s, s + r) for s, r in zip(starts, runs)])
    want = plain.embed(table.double().numpy(), ids, positions, 2.5)
    assert np.abs(plain.sinusoid(positions, hidden)).max() > 0.9  # the position part is as large as the table's
    for s in range(streams):
        np.testing.assert_allclose(x[:8, s], want[:8], atol=2e-4, rtol=0)
        np.testing.assert_allclose(x[8:, s], want[8:], atol=8e-3, rtol=0)  # 40,000 times a rounded frequency
        assert np.array_equal(x[:, s], x[:, 0])


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,streams", [(48, 3), (40, 1), (256, 4), (4100, 2), (72, 8)])
def test_streams_are_written_and_read_in_one_kernel(name, hidden, streams):
    from llm_inference_b200.parts import ops

    dtype, rows = DTYPES[name], 7
    _, _, ctx = context_for({}, dtype, [rows], wanted=[6, 0, 3])
    rng = np.random.default_rng(hidden + streams)
    x = rng.normal(0, 2, (rows, streams, hidden))
    y = rounded(rng.normal(0, 3, (rows, hidden)), dtype)
    mix, out_w, in_w = np.eye(streams) + rng.normal(0, 0.3, (streams, streams)), rng.normal(1, 0.4, streams), rng.normal(0.5, 0.4, streams)
    weight = 1 + rng.normal(0, 0.3, hidden)
    xs = np.moveaxis(x.astype(np.float32).astype(np.float64), 1, 0)
    m32, o32, i32 = (a.astype(np.float32).astype(np.float64) for a in (mix, out_w, in_w))
    w32 = weight.astype(np.float32).astype(np.float64)
    new = plain.streams_write(xs, y.double().numpy(), m32, o32)
    want = plain.rms_norm(plain.streams_read(new, i32), w32, 1e-3)
    x_dev = on_device(x).view(rows, streams * hidden)
    pending = ops.PendingBranch(y.cuda(), on_device(mix), on_device(out_w))
    got = ops.hyper_norm(ctx, x_dev, pending, on_device(in_w), on_device(weight), streams, 1e-3, torch.empty((rows, hidden), dtype=dtype, device="cuda"))
    np.testing.assert_allclose(got.double().cpu().numpy(), want, **CLOSE[name])
    np.testing.assert_allclose(x_dev.cpu().numpy().reshape(rows, streams, hidden), np.moveaxis(new, 0, 1), atol=2e-5, rtol=2e-5)
    # chosen rows, nothing pending, the plain sum of the streams: the model's last norm; the streams stay as they are
    before = x_dev.clone()
    got = ops.hyper_norm(ctx, x_dev, None, None, on_device(weight), streams, 1e-3, torch.empty((3, hidden), dtype=dtype, device="cuda"), ctx.logit_rows)
    np.testing.assert_allclose(got.double().cpu().numpy(), plain.rms_norm(new.sum(axis=0)[[6, 0, 3]], w32, 1e-3), **CLOSE[name])
    # chosen rows with a pending write: the rows are normed as if written, but nothing is stored
    got = ops.hyper_norm(ctx, x_dev, pending, None, on_device(weight), streams, 1e-3, torch.empty((3, hidden), dtype=dtype, device="cuda"), ctx.logit_rows)
    twice = plain.streams_write(new, y.double().numpy(), m32, o32)
    np.testing.assert_allclose(got.double().cpu().numpy(), plain.rms_norm(twice.sum(axis=0)[[6, 0, 3]], w32, 1e-3), **CLOSE[name])
    assert torch.equal(before, x_dev)


def test_soft_cap_of_logits():
    from llm_inference_b200.parts import ops

    _, _, ctx = context_for({}, torch.float32, [3])
    logits = np.random.default_rng(0).normal(0, 40, (3, 1001)).astype(np.float32)
    got = ops.softcap(ctx, torch.from_numpy(logits).cuda(), 30.0).cpu().numpy()
    np.testing.assert_allclose(got, plain.softcap(logits.astype(np.float64), 30.0), atol=1e-5, rtol=1e-6)
    assert np.abs(got).max() < 30.0 and np.abs(logits).max() > 60.0


@pytest.mark.parametrize("experts,groups,keep,top", [(20, 5, 3, 4), (8, 4, 2, 2), (6, 2, 1, 3), (5, 5, 3, 1), (12, 1, 1, 5), (64, 8, 4, 8), (3, 3, 3, 3), (96, 1, 1, 40)])
def test_router_choices_and_weights(experts, groups, keep, top):
    """Random logits, plus rows made so that the largest score of all sits in a group that loses (its
    neighbours are small) while a group of two middling scores wins."""
    from llm_inference_b200.parts import ops

    tokens = 50
    _, _, ctx = context_for({}, torch.float32, [tokens])
    rng = np.random.default_rng(experts * 7 + top)
    logits = rng.normal(0, 2, (tokens, experts)).astype(np.float32)
    size = experts // groups
    if size >= 2 and keep < groups:
        logits[:10] = -3.0 + rng.normal(0, 0.01, (10, experts))
        logits[:10, 0] = 4.0  # alone in group 0: the group scores about 0.98 + 0.05
        for g in range(1, keep + 1):
            logits[:10, g * size : g * size + 2] = 1.0 + rng.normal(0, 0.05, (10, 2))  # about 0.73 + 0.73
    ids = torch.empty((tokens, top), dtype=torch.int32, device="cuda")
    weights = torch.empty((tokens, top), dtype=torch.float32, device="cuda")
    ops.moe_route(ctx, torch.from_numpy(logits).cuda(), groups, keep, top, 2.5, ids, weights)
    ids, weights = ids.cpu().numpy(), weights.cpu().numpy()
    scores = plain.sigmoid(logits.astype(np.float64))
    for t in range(tokens):
        want = plain.route(scores[t], top, groups, keep)
        assert sorted(ids[t]) == sorted(want), f"token {t}"
        np.testing.assert_allclose(weights[t], scores[t, ids[t]] / scores[t, ids[t]].sum() * 2.5, rtol=2e-6)
        if t < 10 and size >= 2 and keep < groups:
            assert 0 not in ids[t]
    assert np.all(np.diff(weights, axis=1) <= 0)  # in the order of the scores


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [dict(), dict(experts=6, top=3, ff=20, groups=(2, 1), shared=(12, 3.0)), dict(experts=5, top=1, ff=70, groups=(5, 3), shared=None),
                                   dict(experts=3, top=2, ff=33, groups=None, limit=0.4), dict(experts=40, top=6, ff=8, groups=(8, 5))])
def test_routed_experts_alone_and_a_token_alone_equals_the_token_in_a_batch(name, sizes):
    from llm_inference_b200.parts import PartSpec, build_part

    dtype, hidden, tokens = DTYPES[name], 48, 150
    mlp = moe(**sizes)
    config = dict(ALPHA, layers=[dict(wkv_layer(), mlp=mlp)])
    weights = {k: v for k, v in draw_weights(config, 31).items() if k.startswith("l0.mlp.")}
    router, shared = mlp["router"], mlp.get("shared")
    groups = router.get("groups") or {"count": 1, "keep": 1}
    part = build_part("feed_forward", PartSpec("routed_experts", dict(
        prefix="l0.mlp.", hidden_size=hidden, experts=router["experts"], top=router["top"], intermediate_size=mlp["expert"]["ff"],
        limit=mlp["expert"]["limit"], route_scale=router["scale"], group_count=groups["count"], group_keep=groups["keep"],
        shared_size=shared["ff"] if shared else None, shared_limit=shared["limit"] if shared else None)))
    part.load(weights, dtype, torch.device("cuda:0"))
    h = rounded(np.random.default_rng(1).normal(0, 1, (tokens, hidden)), dtype)
    want = plain.moe(h.double().numpy(), as_float64(weights), "l0.mlp.", mlp)
    # the clamps bite: without them the result is another
    loose = dict(mlp, expert=dict(mlp["expert"], limit=1e9))
    assert np.abs(plain.moe(h.double().numpy(), as_float64(weights), "l0.mlp.", loose) - want).max() > 0.05
    _, _, ctx = context_for({}, dtype, [tokens])
    got = part.forward(ctx, h.cuda()).clone()
    scale = np.abs(want).max()
    np.testing.assert_allclose(got.double().cpu().numpy() / scale, want / scale, atol=3e-6 if name == "float32" else 2e-2, rtol=0)
    for rows in ([7], [149, 3, 64]):
        _, _, small = context_for({}, dtype, [len(rows)])
        alone = part.forward(small, h[rows].cuda())
        assert torch.equal(alone, got[rows])


@pytest.mark.parametrize("hidden,ff,experts", [(64, 72, 4), (200, 136, 3), (48, 8, 2)])
def test_routed_experts_on_tall_tiles(hidden, ff, experts):
    """bfloat16, 1,100 tokens over a few experts: enough slots per expert that the step sorts them into
    tiles of 128 places, which run on tcgen05 (rows gathered into sorted order, K and output widths that
    are no multiples of the tile sizes). The plain implementation, the FMA kernels and rows fed alone
    (tiles of 32, mma.sync) agree within rounding; with mma.sync for the tall tiles too, rows fed alone
    give the same bits."""
    from llm_inference_b200.parts import PartSpec, build_part

    tokens = 1100
    mlp = moe(experts=experts, top=2, ff=ff, groups=None, shared=(24, 2.0))
    config = dict(ALPHA, width=hidden, layers=[dict(wkv_layer(), mlp=mlp)])
    weights = {k: v for k, v in draw_weights(config, 13).items() if k.startswith("l0.mlp.")}
    part = build_part("feed_forward", PartSpec("routed_experts", dict(
        prefix="l0.mlp.", hidden_size=hidden, experts=experts, top=2, intermediate_size=ff, limit=2.0, route_scale=1.5, shared_size=24, shared_limit=2.0)))
    part.load(weights, torch.bfloat16, torch.device("cuda:0"))
    h = rounded(np.random.default_rng(1).normal(0, 1, (tokens, hidden)), torch.bfloat16)
    want = plain.moe(h.double().numpy(), as_float64(weights), "l0.mlp.", mlp)
    runner, _, ctx = context_for({}, torch.bfloat16, [1])
    ctx.num_tokens = tokens
    got = part.forward(ctx, h.cuda()).clone()
    runner.check()
    scale = np.abs(want).max()
    np.testing.assert_allclose(got.double().cpu().numpy() / scale, want / scale, atol=2e-2, rtol=0)
    ctx.options = dict(ctx.options, moe="plain")
    simple = part.forward(ctx, h.cuda()).clone()
    np.testing.assert_allclose(simple.double().cpu().numpy() / scale, got.double().cpu().numpy() / scale, atol=1e-2, rtol=0)
    ctx.options = dict(ctx.options, moe="mma")
    legacy = part.forward(ctx, h.cuda()).clone()
    np.testing.assert_allclose(legacy.double().cpu().numpy() / scale, got.double().cpu().numpy() / scale, atol=1e-2, rtol=0)
    for rows in ([7], [1099, 3, 640]):
        _, _, small = context_for({}, torch.bfloat16, [len(rows)])
        alone = part.forward(small, h[rows].cuda())
        assert torch.equal(alone, legacy[rows])
        np.testing.assert_allclose(alone.double().cpu().numpy() / scale, got[rows].double().cpu().numpy() / scale, atol=1e-2, rtol=0)


def step_mixers(runner, cache, mixers, portions, inputs):
    """Feed ``portions`` = [(request id, rows of its input)] as one step to the mixer parts, one after the other
    (cache entry i for mixer i); returns each mixer's output rows by request."""
    from llm_inference_b200.engine.runner import StepEntry

    sizes = [rows.stop - rows.start for _, rows in portions]
    entries = [StepEntry(rid, [0] * size) for (rid, _), size in zip(portions, sizes)]
    order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) != 1, i))  # single tokens lead a batch
    entries = [entries[i] for i in order]
    starts = [cache.manager.length(e.request_id) for e in entries]
    for e, s in zip(entries, starts):
        cache.manager.ensure(e.request_id, s + len(e.tokens))
    cache.clear_new_slots()
    ctx = runner._build_context(entries, starts, [])
    h = torch.cat([inputs[portions[i][0]][portions[i][1]] for i in order]).cuda()
    outs = [mixer.forward(ctx, cache.view(index, True, runner._tables), h).clone() for index, mixer in enumerate(mixers)]
    for e, s in zip(entries, starts):
        cache.manager.advance(e.request_id, s + len(e.tokens))
    results = []
    for out in outs:
        result, row = {}, 0
        for i in order:
            result[portions[i][0]] = out[row : row + sizes[i]].double().cpu().numpy()
            row += sizes[i]
        results.append(result)
    return results


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [dict(), dict(heads=1, dim=6, decay_rank=2), dict(heads=2, dim=40, decay_rank=3), dict(heads=3, dim=130, decay_rank=4)])
def test_recurrent_mixer_alone_in_portions_beside_another_request(name, sizes):
    """The matrix state and the previous token's input carry across steps of 5, 1, 2, 1, ... tokens; a
    second request moves through another slot at the same time. The slowest channels keep the first
    token in the state to the end: without it the last read-outs differ visibly; so does the bonus."""
    from llm_inference_b200.parts import PartSpec, build_part

    dtype, hidden, total = DTYPES[name], 48, 41
    config = dict(ALPHA, layers=[dict(wkv_layer(**sizes), mlp=None)])
    m = config["layers"][0]["mixer"]
    weights = {k: v for k, v in draw_weights(config, 5).items() if k.startswith("l0.mix.")}
    w64 = as_float64(weights)
    mixer = build_part("mixer", PartSpec("wkv", dict(prefix="l0.mix.", hidden_size=hidden, heads=m["heads"], dim=m["dim"], eps=1e-5)))
    rng = np.random.default_rng(2)
    inputs = {10: rounded(rng.normal(0, 1, (total, hidden)), dtype), 11: rounded(rng.normal(0, 1, (12, hidden)), dtype)}
    want = {rid: plain.wkv_mixer(rows.double().numpy(), w64, "l0.mix.", m["heads"], m["dim"], 1e-5)[0] for rid, rows in inputs.items()}
    headless = plain.wkv_mixer(inputs[10].double().numpy()[1:], w64, "l0.mix.", m["heads"], m["dim"], 1e-5)[0]
    assert np.abs(headless[-10:] - want[10][-10:]).max() > 1e-2
    no_bonus = plain.wkv_mixer(inputs[10].double().numpy(), dict(w64, **{"l0.mix.u": np.zeros((m["heads"], m["dim"]))}), "l0.mix.", m["heads"], m["dim"], 1e-5)[0]
    assert np.abs(no_bonus - want[10]).max() > 1e-1
    mixer.load(weights, dtype, torch.device("cuda:0"))
    runner, cache, _ = context_for({0: mixer.cache_spec()}, dtype, [1])
    for arrays in cache.states.values():
        for array in arrays:
            array.fill_(float("nan"))  # a slot is cleared when it is handed out, not before
    cache.open(10), cache.open(11)
    got = {10: [], 11: []}
    at, other = 0, 0
    for portion in (5, 1, 2, 1, 1, 17, 3, 1, 10):
        step = [(10, slice(at, at + portion))]
        if other < 12:
            size = 1 if other % 2 else 3
            step.append((11, slice(other, other + size)))
            other += size
        (out,) = step_mixers(runner, cache, [mixer], step, inputs)
        for rid in out:
            got[rid].append(out[rid])
        at += portion
    runner.check()
    assert at == total and other == 12
    tolerance = dict(CLOSE[name], atol=CLOSE[name]["atol"] * 3)
    np.testing.assert_allclose(np.concatenate(got[10]), want[10], **tolerance)
    np.testing.assert_allclose(np.concatenate(got[11]), want[11], **tolerance)


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [dict(), dict(heads=5, kv_heads=1, dim=72, vdim=40, scale=0.7), dict(heads=3, kv_heads=3, dim=8, vdim=136, scale=3.0),
                                   dict(heads=6, kv_heads=2, dim=64, vdim=64, scale=0.8), dict(heads=4, kv_heads=4, dim=128, vdim=128, scale=0.5)])
def test_gated_attention_alone_and_with_blended_values_in_portions(name, sizes):
    """Two layers over the same inputs, the second blending its values with the first's: 70 tokens over
    pages of 8 in portions that end before, on and after page borders, beside a second request. Scores
    are sharp enough that single keys, near and far, carry the output: the last queries' output
    without the keys of the first page is far outside the tolerance, and so is the output without the
    gate or without the blend."""
    from llm_inference_b200.parts import PartSpec, build_part

    dtype, hidden, total = DTYPES[name], 48, 70
    config = dict(ALPHA, layers=[dict(attention_layer(**sizes, v_mix=True), mlp=None), dict(attention_layer(**sizes, v_mix=True), mlp=None)])
    m = config["layers"][0]["mixer"]
    weights = {k: v for k, v in draw_weights(config, 21).items() if ".mix." in k}
    w64 = as_float64(weights)

    def build(index, values):
        return build_part("mixer", PartSpec("gated_attention", dict(
            prefix=f"l{index}.mix.", hidden_size=hidden, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], scale=m["scale"],
            eps=1e-5, values=values)))

    mixers = [build(0, "publish"), build(1, "blend")]
    rng = np.random.default_rng(8)
    inputs = {10: rounded(rng.normal(0, 1, (total, hidden)), dtype), 11: rounded(rng.normal(0, 1, (9, hidden)), dtype)}

    def reference(rows, first=0, blend=True):
        out0, _, raw = plain.attention_mixer(rows, w64, "l0.mix.", m, 1e-5, first)
        out1, _, _ = plain.attention_mixer(rows, w64, "l1.mix.", m, 1e-5, first, None, raw, blend)
        return out0, out1

    want = {rid: reference(rows.double().numpy()) for rid, rows in inputs.items()}
    shifted = reference(inputs[10].double().numpy()[8:])
    assert np.abs(shifted[0][-20:] - want[10][0][-20:]).max() > 0.3  # keys 50 and more positions back carry the last queries
    assert np.abs(reference(inputs[10].double().numpy(), blend=False)[1] - want[10][1]).max() > 0.1
    runner, cache, _ = context_for({0: mixers[0].cache_spec(), 1: mixers[1].cache_spec()}, dtype, [1])
    for group in cache.groups:
        group.arena.fill_(float("nan"))  # pages are not cleared between requests: a request reads only what it wrote
    for mixer in mixers:
        mixer.load(weights, dtype, torch.device("cuda:0"))
    cache.open(10), cache.open(11)
    got = {10: ([], []), 11: ([], [])}
    at, other = 0, 0
    for portion in (7, 1, 2, 30, 1, 1, 8, 20):
        step = [(10, slice(at, at + portion))]
        if other < 9:
            step.insert(0, (11, slice(other, other + (1 if other else 3))))
        outs = step_mixers(runner, cache, mixers, step, inputs)
        for layer, out in enumerate(outs):
            for rid in out:
                got[rid][layer].append(out[rid])
        at += portion
        other += (1 if other else 3) if other < 9 else 0
    runner.check()
    assert at == total
    for layer in range(2):
        np.testing.assert_allclose(np.concatenate(got[10][layer]), want[10][layer], **CLOSE[name])
        np.testing.assert_allclose(np.concatenate(got[11][layer]), want[11][layer][: sum(len(g) for g in got[11][layer])], **CLOSE[name])


# --- whole models ---------------------------------------------------------------------------------------------


LENGTHS = [1, 2, 3, 9, 31, 70, 150]


@pytest.fixture(scope="module", params=["alpha", "beta", "gamma"])
def model_case(request, tmp_path_factory):
    config = CONFIGS[request.param]
    weights = draw_weights(config, seed=17 + len(request.param))
    folder = write_folder(tmp_path_factory.mktemp(request.param), config, weights)
    rng = np.random.default_rng(4)
    sequences = {f"s{n}": [int(t) for t in rng.integers(0, config["vocab"], n)] for n in LENGTHS}
    w64 = as_float64(weights)
    expected = {key: plain.forward(config, w64, tokens) for key, tokens in sequences.items()}
    return request.param, config, folder, sequences, expected, w64


# A router's choice is a step function of its scores: where two candidates are closer than bfloat16
# rounding moves them, the engine may rightly choose the other one, and that token's logits (and, through
# the cache and the recurrent state, later ones) then differ by much more than rounding. So in
# bfloat16 the plain implementation is run a second time along the engine's own choices, which every
# routed layer leaves in a buffer of its own, and each choice that differs from the plain one must
# have been a close call in that run. In float32 the plain implementation's own choices stand.
CLOSE_CALL = 0.03


class RoutedReplay(Replay):
    """A replay that also files every routed layer's choices by (request, layer, position)."""

    def __init__(self, config, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.routed = {i: layer["mlp"]["router"]["top"] for i, layer in enumerate(config["layers"]) if layer.get("mlp") is not None}
        self.chosen: dict[tuple[str, int, int], np.ndarray] = {}

    def step(self, portions, end=()):
        before = {name: self.at.get(name, 0) for name, _ in portions}
        super().step(portions, end)
        order = sorted(range(len(portions)), key=lambda i: (len(portions[i][1]) != 1, i))  # single tokens lead a batch
        for layer, top in self.routed.items():
            flat = self.runner.workspace._flat[f"moe_ids:l{layer}.mlp.:torch.int32"].cpu().numpy()
            row = 0
            for i in order:
                name, tokens = portions[i]
                for j in range(len(tokens)):
                    self.chosen[(name, layer, before[name] + j)] = flat[row * top : (row + 1) * top].copy()
                    row += 1

    def choices(self, name: str, length: int) -> dict[int, np.ndarray]:
        return {layer: np.stack([self.chosen[(name, layer, i)] for i in range(length)]) for layer in self.routed}


def expected_along(case, replay, key: str, tokens, dtype: str) -> np.ndarray:
    """The plain logits for ``tokens``: in bfloat16 along the engine's choices of experts, which may differ
    from the plain ones only where the plain run saw a close call."""
    _, config, _, _, expected, w64 = case
    if dtype == "float32":
        return expected[key] if key in expected else plain.forward(config, w64, tokens)
    choices = replay.choices(key, len(tokens))
    margins, free = [], []
    logits = plain.forward(config, w64, tokens, margins=margins, choices=choices, free=free)
    differing = 0
    for at, layer in enumerate(sorted(choices)):
        for t in range(len(tokens)):
            if set(choices[layer][t].tolist()) != set(free[at][t].tolist()):
                differing += 1
                assert margins[at][t] < CLOSE_CALL, f"request {key}, layer {layer}, position {t}: the engine chose {choices[layer][t]}, plain {free[at][t]} by {margins[at][t]:.3f}"
    assert differing <= 0.1 * max(1, len(choices)) * len(tokens) + 1
    return logits


def check_all(case, replay, sequences, dtype: str, what: str) -> None:
    errors = []
    for key, tokens in sequences.items():
        error = row_error(replay.of(key, len(tokens)), expected_along(case, replay, key, tokens, dtype))
        assert error.max() <= TOLERANCE[dtype], f"{what}: request {key}, position {int(error.argmax())}: error {error.max():.2e}"
        errors.append(error)
    mean = np.concatenate(errors).mean()
    assert mean <= MEAN_TOLERANCE[dtype], f"{what}: mean error over all rows {mean:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_one_by_one_against_plain(model_case, dtype):
    """The sum of the streams after every layer of a short prompt, so that a fault names its layer."""
    from llm_inference_b200.engine.runner import StepEntry

    _, config, folder, sequences, _, w64 = model_case
    tokens = sequences["s31"]
    replay = RoutedReplay(config, folder, dtype, 64)
    replay.cache.open(1)
    replay.cache.manager.ensure(1, len(tokens))
    replay.cache.clear_new_slots()
    ctx = replay.runner._build_context([StepEntry(1, tokens)], [0], [])
    x = replay.model.embedding.forward(ctx)
    n = config.get("streams") or 1
    pending, sums, choices = None, [], {}
    for index, call in enumerate(replay.model.schedule):
        block = replay.model.blocks[call.layer]
        pending = block.forward(ctx, replay.runner._view(call, replay.runner._tables), x, pending)
        streams = x.double().view(len(tokens), n, -1)
        written = torch.einsum("sr,tsd->trd", pending.mix.double(), streams) + pending.out.double()[None, :, None] * pending.y.double()[:, None, :]
        sums.append(written.sum(dim=1).cpu().numpy())
        if block.feed_forward is not None:
            choices[index] = ctx.buffer(f"moe_ids:l{index}.mlp.", (len(tokens), block.feed_forward.top), torch.int32).cpu().numpy()
    replay.runner.check()
    layers: list = []
    plain.forward(config, w64, tokens, layer_sums=layers, choices=None if dtype == "float32" else choices)
    for index, (got, want) in enumerate(zip(sums, layers)):
        error = np.abs(got - want).max() / np.abs(want).max()
        assert error <= (1e-5 if dtype == "float32" else 6e-2), f"layer {index} ({config['layers'][index]['type']}): {error:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_one_after_another_in_a_pool_for_one(model_case, dtype):
    _, config, folder, sequences, _, _ = model_case
    replay = RoutedReplay(config, folder, dtype, 152, slots=1)
    for key, tokens in sequences.items():
        replay.step([(key, tokens)], end=(key,))
    check_all(model_case, replay, sequences, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token(model_case, dtype):
    """All but the last 40 tokens as one portion, the rest one by one (captured steps replayed)."""
    _, config, folder, sequences, _, _ = model_case
    replay = RoutedReplay(config, folder, dtype, 152, slots=1)
    for key, tokens in sequences.items():
        head = max(0, len(tokens) - 40)
        if head:
            replay.step([(key, tokens[:head])])
        for position in range(head, len(tokens)):
            replay.step([(key, [tokens[position]])], end=(key,) if position == len(tokens) - 1 else ())
    check_all(model_case, replay, sequences, dtype, "token by token")
    assert replay.runner.graph_replays > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2,), (3, 1, 2, 8, 1, 17), (7, 9, 64)])
def test_portions_of_changing_size(model_case, dtype, sizes):
    _, config, folder, sequences, _, _ = model_case
    replay = RoutedReplay(config, folder, dtype, 152, slots=1)
    for key, tokens in sequences.items():
        at, turn = 0, 0
        while at < len(tokens):
            size = min(sizes[turn % len(sizes)], len(tokens) - at)
            replay.step([(key, tokens[at : at + size])], end=(key,) if at + size == len(tokens) else ())
            at, turn = at + size, turn + 1
    check_all(model_case, replay, sequences, dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(model_case, dtype):
    """Up to three live requests (three slots, 38 pages of 8 for sequences that need 46 in all): portions
    of some beside single tokens of others, requests left out of steps, and every request that
    ends hands its pages and its slot to one that starts later."""
    _, config, folder, sequences, _, _ = model_case
    replay = RoutedReplay(config, folder, dtype, 304, slots=3)
    rng = np.random.default_rng(9)
    waiting = ["s150", "s70", "s31", "s9", "s3", "s2", "s1", "again70", "again9"]
    sequences = dict(sequences, again70=sequences["s70"], again9=sequences["s9"])
    live: dict[str, int] = {}
    while waiting or live:
        while waiting and len(live) < 3:
            live[waiting.pop(0)] = 0
        portions, end = [], []
        for key in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            left = len(sequences[key]) - live[key]
            size = min(left, int(rng.choice([1, 1, 1, 2, 3, 8, 29])))
            portions.append((key, sequences[key][live[key] : live[key] + size]))
            live[key] += size
            if live[key] == len(sequences[key]):
                end.append(key)
                del live[key]
        if portions:
            replay.step(portions, end=tuple(end))
    check_all(model_case, replay, sequences, dtype, "mixed")
    stats = replay.cache.stats()
    assert stats["free_state_slots"] == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_case, dtype):
    """Four tokens of prompt, then 330 single tokens: the recurrent state and the cache after hundreds
    of steps, across many pages."""
    _, config, folder, _, _, w64 = model_case
    tokens = [int(t) for t in np.random.default_rng(6).integers(0, config["vocab"], 334)]
    replay = RoutedReplay(config, folder, dtype, 384, slots=1)
    replay.step([("long", tokens[:4])])
    for token in tokens[4:]:
        replay.step([("long", [token])])
    error = row_error(replay.of("long", len(tokens)), expected_along(model_case, replay, "long", tokens, dtype))
    assert error.max() <= TOLERANCE[dtype], f"position {int(error.argmax())}: {error.max():.2e}"
    assert error.mean() <= MEAN_TOLERANCE[dtype] and error[-50:].mean() <= MEAN_TOLERANCE[dtype], f"mean {error.mean():.2e}, last 50 {error[-50:].mean():.2e}"
    assert replay.runner.graph_replays > 300


def test_trace_tool_mixed_schedule(model_case, tmp_path):
    """bin/trace_run itself: two requests interleaved, a third that reuses what the first gave back."""
    _, config, folder, sequences, expected, _ = model_case
    a, b, c = sequences["s70"], sequences["s31"], sequences["s9"]
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 32]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:2], "want": [1]}, {"id": "a", "tokens": a[33:34], "want": [0]}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[34:], "want": [35]}, {"id": "b", "tokens": b[2:3], "want": []}], "end": ["a"]},
        {"step": 3, "entries": [{"id": "b", "tokens": b[3:], "want": [27]}, {"id": "c", "tokens": c, "want": [8]}], "end": ["b", "c"]},
    ]
    want = [expected["s70"][[0, 32]], expected["s31"][[1]], expected["s70"][[33]], expected["s70"][[69]], expected["s31"][[30]], expected["s9"][[8]]]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        result = subprocess.run(
            [sys.executable, str(TRACE_RUN), "--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", "256"],
            input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600,
        )
        assert result.returncode == 0, result.stderr[-3000:]
        assert [line for line in result.stdout.splitlines() if line.startswith("done ")] == [f"done {i}" for i in range(4)]
        got = np.concatenate([np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, config["vocab"]) for i in range(4)])
        error = row_error(got, np.concatenate(want))
        if dtype == "float32":
            assert error.max() <= TOLERANCE[dtype]
        else:  # the tool gives no routing choices to follow: all but a row that met a close call are within the bound
            assert np.sort(error)[-2] <= TOLERANCE[dtype]


def test_greedy_generation_through_the_engine(model_case):
    """submit / step / sample through the scheduler: float32 gives the plain implementation's tokens;
    two requests at once give what each gives alone."""
    from llm_inference_b200 import create_engine

    _, config, folder, sequences, _, w64 = model_case
    prompt, other = sequences["s31"], sequences["s9"]
    want = plain.greedy(config, w64, prompt, 12)
    with create_engine(folder, dtype="float32", max_num_sequences=3, max_model_length=128, kv_cache_bytes=4 << 20, page_size=8,
                       prefill_chunk_size=16, prefill_burst_size=16) as engine:
        assert engine.generate(prompt, 12) == want
        first, second = engine.submit(prompt, 12), engine.submit(other, 7)
        while engine.has_work():
            engine.step()
        assert engine.request(first).output == want
        assert engine.request(second).output == plain.greedy(config, w64, other, 7)
        assert engine.stats()["free_state_slots"] == 3
    with create_engine(folder, dtype="bfloat16", max_num_sequences=2, max_model_length=128, kv_cache_bytes=4 << 20, page_size=8) as engine:
        got = engine.generate(prompt, 12)
    tokens = list(prompt)
    for token in got:  # only a near-tie may go the other way in bfloat16
        row = plain.forward(config, w64, tokens)[-1]
        if token != int(np.argmax(row)):
            assert row.max() - row[token] <= 0.1 * row.std()
            break
        tokens.append(token)


def test_command_line_tools_take_the_design(tmp_path):
    """A seeded folder from the named shape, its inspection, and greedy generation from the folder and from
    the shape itself (weights drawn on the device)."""
    run = lambda *args: subprocess.run([sys.executable, "-m", *args], capture_output=True, text=True, timeout=600)
    folder = tmp_path / "model"
    made = run("llm_inference_b200.cli.random_model", "--preset", "tunadra-small", "--seed", "3", "--out", str(folder))
    assert made.returncode == 0, made.stderr[-2000:]
    seen = run("llm_inference_b200.cli.inspect_model", str(folder))
    assert seen.returncode == 0 and "architecture: Tunadra" in seen.stdout and "l1.mix.w0" in seen.stdout, seen.stderr[-2000:]
    ask = ["--prompt-ids", "5,17,3,900,41", "--max-new-tokens", "6", "--max-model-length", "256", "--kv-cache-mib", "64"]
    from_folder = run("llm_inference_b200.cli.generate", "--model", str(folder), *ask)
    from_shape = run("llm_inference_b200.cli.generate", "--random", "tunadra-small", "--weights-seed", "3", *ask)
    assert from_folder.returncode == 0, from_folder.stderr[-2000:]
    assert from_shape.returncode == 0, from_shape.stderr[-2000:]
    for result in (from_folder, from_shape):
        line = json.loads(result.stdout.strip().splitlines()[-1])
        assert line["prompt_tokens"] == 5 and len(line["tokens"]) == 6 and all(0 <= t < 8192 for t in line["tokens"])
