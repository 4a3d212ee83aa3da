"""Gunedra: every mechanism alone against the plain implementation, then whole models in every
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

from gunedra_helpers import ALPHA, BETA, CONFIGS, MEAN_TOLERANCE, TOLERANCE, Replay, as_float64, delta_mixer, draw_weights, latent_mixer, row_error, write_folder
from helpers import TRACE_RUN
from plain import gunedra_plain as plain
from test_parts import context_for

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CLOSE = {"float32": dict(atol=2e-5, rtol=2e-5), "bfloat16": dict(atol=5e-2, rtol=3e-2)}


def rounded(array: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(array)).to(dtype)


# --- kernels and parts alone ---------------------------------------------------------------------------


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,groups", [(48, 4), (40, 1), (192, 3), (4100, 2)])
def test_branch_norm_add_with_and_without_depth_mix(name, hidden, groups):
    from llm_inference_b200.parts import ops

    dtype, rows, depth = DTYPES[name], 7, 4
    _, _, ctx = context_for({}, dtype, [rows])
    rng = np.random.default_rng(hidden)
    x = rng.normal(0, 2, (rows, hidden)).astype(np.float32)
    branch = rounded(rng.normal(0, 3, (rows, hidden)), dtype)
    weight, scale = (1 + rng.normal(0, 0.3, hidden)).astype(np.float32), rng.normal(1, 0.3, hidden).astype(np.float32)
    history = rng.normal(0, 1, (depth, rows, hidden)).astype(np.float32)
    mix = rng.uniform(0.1, 1.0, depth).astype(np.float32)
    normed = plain.grouped_rms_norm(branch.double().numpy(), weight.astype(np.float64), groups, 1e-3)
    want = x.astype(np.float64) + 0.7 * scale * normed
    d = lambda a: torch.from_numpy(a).cuda()
    x_in, hist = d(x), d(history)
    mixed, copy = torch.empty_like(x_in), torch.empty_like(x_in)
    cast = torch.empty((rows, hidden), dtype=dtype, device="cuda")
    ops.branch_norm_add(ctx, x_in, branch.cuda(), d(weight), d(scale), 0.7, groups, 1e-3, hist[depth - 1], copy_in=copy, history=hist,
                        mix=d(mix), mixed=mixed, cast=cast)
    want_mixed = sum(mix[j].astype(np.float64) * history[j] for j in range(depth - 1)) + mix[depth - 1] * want
    np.testing.assert_allclose(hist[depth - 1].cpu().numpy(), want, **CLOSE["float32"])
    np.testing.assert_allclose(mixed.cpu().numpy(), want_mixed, **CLOSE["float32"])
    np.testing.assert_allclose(cast.double().cpu().numpy(), want_mixed, **CLOSE[name])
    assert torch.equal(copy, x_in)
    # without a mix, in place, no scale: the rounded copy is the stream itself
    ops.branch_norm_add(ctx, x_in, branch.cuda(), d(weight), None, 1.5, groups, 1e-3, x_in, cast=cast)
    np.testing.assert_allclose(x_in.cpu().numpy(), x + 1.5 * normed, **CLOSE["float32"])
    np.testing.assert_allclose(cast.double().cpu().numpy(), x + 1.5 * normed, **CLOSE[name])


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
def test_grouped_norm_of_chosen_rows_poly_norm_and_scaled_embedding(name):
    from llm_inference_b200.parts import PartSpec, build_part, ops

    dtype, hidden, vocab, tokens = DTYPES[name], 60, 37, 9
    _, _, ctx = context_for({}, dtype, [tokens], wanted=[8, 0, 3])
    rng = np.random.default_rng(3)
    norm = build_part("norm", PartSpec("grouped_rmsnorm", dict(name="n", hidden_size=hidden, groups=5, eps=1e-4)))
    embedding = build_part("embedding", PartSpec("token_embedding", dict(name="e", suffix="", vocab_size=vocab, hidden_size=hidden, scale=2.5, cast=True)))
    weights = {"n": rounded(1 + rng.normal(0, 0.3, hidden), torch.bfloat16), "e": rounded(rng.normal(0, 1, (vocab, hidden)), torch.bfloat16)}
    norm.load(weights, dtype, ctx.device), embedding.load(weights, dtype, ctx.device)
    ids = rng.integers(0, vocab, tokens)
    ctx.token_ids.copy_(torch.from_numpy(ids.astype(np.int32)).cuda())
    x = embedding.forward(ctx)
    want_x = plain.embed(weights["e"].double().numpy(), ids, 2.5)
    np.testing.assert_allclose(x.cpu().numpy(), want_x, **CLOSE["float32"])
    if dtype != torch.float32:
        np.testing.assert_allclose(ctx.buffer("stream_cast", (tokens, hidden)).double().cpu().numpy(), want_x, **CLOSE[name])
    rows = norm.forward(ctx, x, None, rows=ctx.logit_rows, out_name="rows")
    want = plain.grouped_rms_norm(want_x[[8, 0, 3]], weights["n"].double().numpy(), 5, 1e-4)
    np.testing.assert_allclose(rows.double().cpu().numpy(), want, **CLOSE[name])
    # PolyNorm with coefficients that make every power matter
    z = rounded(rng.normal(0, 1.5, (tokens, 200)), dtype)
    coefficients = np.array([0.8, -0.5, 0.3, 0.1], dtype=np.float32)
    got = ops.poly_norm(ctx, z.cuda(), torch.from_numpy(coefficients).cuda(), 1e-5, torch.empty_like(z, device="cuda"))
    zz = z.double().numpy()
    want = sum(c * (zz**p) / plain.rms(zz**p, 1e-5) for c, p in zip(coefficients[:3].astype(np.float64), (1, 2, 3))) + 0.1
    np.testing.assert_allclose(got.double().cpu().numpy(), want, **CLOSE[name])


def step_mixer(runner, cache, mixer, cache_id, portions, inputs):
    """Feed ``portions`` = [(request id, rows of its input)] as one step to a mixer part."""
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
    out = mixer.forward(ctx, cache.view(cache_id, True, runner._tables), h).clone()
    for e, s in zip(entries, starts):
        cache.manager.advance(e.request_id, s + len(e.tokens))
    result, row = {}, 0
    for i in order:
        result[portions[i][0]] = out[row : row + sizes[i]].double().cpu().numpy()
        row += sizes[i]
    return result


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [dict(), dict(heads=5, dim=12, rot_dim=12, vdim=6, kv_rank=72, rot_dims=8, base=1e5, scale=0.31)])
def test_latent_attention_alone_in_portions_beside_another_request(name, sizes):
    """70 tokens over pages of 8 in portions that end before, on and after page borders, beside a
    second request; queries sharp enough that single keys, near and far, carry the output, and
    sinks that carry a share of it: the plain output without the sink, and the last queries'
    output without the keys of the first page, are both far outside the tolerance."""
    from llm_inference_b200.parts import PartSpec, build_part

    dtype, hidden, total = DTYPES[name], 48, 70
    config = dict(ALPHA, layers=[dict(latent_mixer(**sizes), mlp=None)])
    m = config["layers"][0]["mixer"]
    weights = {k: v for k, v in draw_weights(config, 21, sharp=6.0).items() if k.startswith("l0.mix.")}
    w64 = as_float64(weights)
    mixer = build_part("mixer", PartSpec("latent_attention", dict(
        prefix="l0.mix.", hidden_size=hidden, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], rank=m["kv_rank"],
        scale=m["scale"], eps=1e-5, position=PartSpec("rotary", dict(head_dim=m["rot_dim"], theta=m["rot"]["base"], rotary_dims=m["rot"]["dims"], interleaved=True)))))
    rng = np.random.default_rng(8)
    inputs = {10: rounded(rng.normal(0, 1, (total, hidden)), dtype), 11: rounded(rng.normal(0, 1, (9, hidden)), dtype)}
    want = {rid: plain.latent_attention(config, w64, "l0.mix.", m, rows.double().numpy(), np.arange(len(rows))) for rid, rows in inputs.items()}
    # the construction shows what it is meant to show
    no_sink = plain.latent_attention(config, dict(w64, **{"l0.mix.sink": np.full(m["heads"], -1e9)}), "l0.mix.", m, inputs[10].double().numpy(), np.arange(total))
    assert np.abs(no_sink - want[10]).max() > 0.5
    shifted = plain.latent_attention(config, w64, "l0.mix.", m, inputs[10].double().numpy()[8:], np.arange(8, total))
    assert np.abs(shifted[-20:] - want[10][-20:]).max() > 0.5  # keys 50 and more positions back carry the last queries

    runner, cache, _ = context_for({0: mixer.cache_spec()}, dtype, [1])
    mixer.load(weights, dtype, torch.device("cuda:0"))
    cache.open(10), cache.open(11)
    got = {10: [], 11: []}
    at, other = 0, 0
    for portion in (7, 1, 2, 30, 1, 1, 8, 20):
        step = [(10, slice(at, at + portion))]
        if other < 9:
            step.insert(0, (11, slice(other, other + (1 if other else 3))))
        out = step_mixer(runner, cache, mixer, 0, step, inputs)
        for rid in out:
            got[rid].append(out[rid])
        at += portion
        other += (1 if other else 3) if other < 9 else 0
    runner.check()
    assert at == total
    np.testing.assert_allclose(np.concatenate(got[10]), want[10], **CLOSE[name])
    np.testing.assert_allclose(np.concatenate(got[11]), want[11][: sum(len(g) for g in got[11])], **CLOSE[name])


@pytest.mark.parametrize("name", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [dict(), dict(heads=2, kv_heads=1, dim=40, vdim=8, conv=4), dict(heads=1, kv_heads=1, dim=16, vdim=36, conv=1),
                                   dict(heads=3, kv_heads=3, dim=4, vdim=130, conv=2)])
def test_delta_rule_alone_in_portions_beside_another_request(name, sizes):
    """The state and the convolution's last inputs carry across steps of 5, 1, 2, 1, ... tokens;
    a second request moves through another slot at the same time. The slowest head's decay keeps
    the first token in the state to the end: without it the last read-outs differ visibly."""
    from llm_inference_b200.parts import PartSpec, build_part

    dtype, hidden, total = DTYPES[name], 48, 41
    config = dict(ALPHA, layers=[dict(delta_mixer(**sizes), mlp=None)])
    m = config["layers"][0]["mixer"]
    weights = {k: v for k, v in draw_weights(config, 5).items() if k.startswith("l0.mix.")}
    w64 = as_float64(weights)
    mixer = build_part("mixer", PartSpec("channel_delta", dict(
        prefix="l0.mix.", hidden_size=hidden, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], taps=m["conv"], eps=1e-5)))
    rng = np.random.default_rng(2)
    inputs = {10: rounded(rng.normal(0, 1, (total, hidden)), dtype), 11: rounded(rng.normal(0, 1, (12, hidden)), dtype)}
    want = {rid: plain.channel_delta(config, w64, "l0.mix.", m, rows.double().numpy()) for rid, rows in inputs.items()}
    assert np.abs(plain.channel_delta(config, w64, "l0.mix.", m, inputs[10].double().numpy()[1:])[-10:] - want[10][-10:]).max() > 1e-2
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
        out = step_mixer(runner, cache, mixer, 0, step, inputs)
        for rid in out:
            got[rid].append(out[rid])
        at += portion
    runner.check()
    assert at == total and other == 12
    tolerance = dict(CLOSE[name], atol=CLOSE[name]["atol"] * 3)
    np.testing.assert_allclose(np.concatenate(got[10]), want[10], **tolerance)
    np.testing.assert_allclose(np.concatenate(got[11]), want[11], **tolerance)


@pytest.mark.parametrize("heads,rank,rot_dim", [(3, 64, 16), (5, 160, 32), (6, 128, 32), (12, 512, 64), (40, 96, 16), (1, 32, 0)])
def test_tensor_core_latent_attention_against_the_plain_kernel(heads, rank, rot_dim):
    """bfloat16: three single tokens (a request's very first token, one at a page border, one far in)
    and three prompt portions (from the start, deep in a request, across many pages) in one step; the
    pages hold NaN wherever the requests have not written, queries are sharp, sinks and gates matter.
    The keys of single tokens are cut into 1, 3 and the default number of pieces."""
    from llm_inference_b200.parts import ops
    from llm_inference_b200.parts.base import KVCacheSpec

    from llm_inference_b200.engine.runner import StepEntry

    runs, starts = [1, 1, 1, 37, 5, 70], [0, 63, 150, 0, 90, 31]
    runner, cache, _ = context_for({0: KVCacheSpec(1, rank + rot_dim, 0, planes=1)}, torch.bfloat16, [1])
    entries = []
    for i, (run, start) in enumerate(zip(runs, starts)):
        cache.open(10 + i)
        cache.manager.ensure(10 + i, start + run)
        cache.manager.advance(10 + i, start)
        entries.append(StepEntry(10 + i, [0] * run))
    ctx = runner._build_context(entries, starts, [])
    assert ops.latent_attention_mma_supported(ctx, heads, rank, rot_dim, cache.page_size) and ctx.num_decode_seqs == 3
    view = cache.view(0, True, runner._tables)
    generator = torch.Generator(device="cuda").manual_seed(heads * 1000 + rank)
    normal = lambda *shape: torch.randn(*shape, device="cuda", generator=generator)
    view.keys.fill_(float("nan"))
    table = runner._tables[0].cpu().numpy()
    for i, (run, start) in enumerate(zip(runs, starts)):
        for j in range(start + run):
            view.keys[int(table[i, j // 8]), 0, j % 8] = normal(rank + rot_dim).to(torch.bfloat16)
    tokens = sum(runs)
    q_lat = (normal(heads, tokens, rank) * 3.0 / rank**0.5).to(torch.bfloat16)
    q_rot = (normal(tokens, heads * rot_dim) * 0.5).to(torch.bfloat16)
    sink = normal(heads) + 1.5
    gate = normal(tokens, heads + 3).to(torch.bfloat16)[:, 1 : heads + 1]  # a slice of wider rows, as in the mixer
    want = torch.empty(heads, tokens, rank, dtype=torch.bfloat16, device="cuda")
    ops.latent_attention_plain(ctx, view, q_lat, q_rot, sink, gate, want, heads, rank, rot_dim, 0.9)
    assert torch.isfinite(want).all() and want.float().std() > 0.05
    for pieces in (1, 3, 0):
        got = torch.full_like(want, float("nan"))
        if pieces:
            ops.latent_attention_mma(ctx, view, q_lat, q_rot, sink, gate, got, heads, rank, rot_dim, 0.9, first_seq=0, num_seqs=3, max_q_len=1, pieces=pieces)
            ops.latent_attention_mma(ctx, view, q_lat, q_rot, sink, gate, got, heads, rank, rot_dim, 0.9, first_seq=3, num_seqs=3, max_q_len=70)
        else:
            from llm_inference_b200.parts import attention_dispatch

            attention_dispatch.attend_latent(ctx, view, q_lat, q_rot, sink, gate, got, heads, rank, rot_dim, 0.9)
        runner.check()
        np.testing.assert_allclose(got.float().cpu().numpy(), want.float().cpu().numpy(), atol=2e-2, rtol=2e-2, err_msg=f"pieces {pieces}")
    # without sink and gate
    ops.latent_attention_plain(ctx, view, q_lat, q_rot, None, None, want, heads, rank, rot_dim, 0.9)
    got = torch.full_like(want, float("nan"))
    ops.latent_attention_mma(ctx, view, q_lat, q_rot, None, None, got, heads, rank, rot_dim, 0.9, first_seq=0, num_seqs=6, max_q_len=70)
    np.testing.assert_allclose(got.float().cpu().numpy(), want.float().cpu().numpy(), atol=2e-2, rtol=2e-2)


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


def check_all(replay: Replay, sequences, expected, dtype: str, what: str) -> None:
    errors = []
    for key, tokens in sequences.items():
        error = row_error(replay.of(key, len(tokens)), expected[key])
        assert error.max() <= TOLERANCE[dtype], f"{what}: request {key}, position {int(error.argmax())}: error {error.max():.2e}"
        errors.append(error)
    mean = np.concatenate(errors).mean()
    assert mean <= MEAN_TOLERANCE[dtype], f"{what}: mean error over all rows {mean:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_one_by_one_against_plain(model_case, dtype):
    """The stream after every layer of a short prompt, so that a fault names its layer."""
    from llm_inference_b200.engine.runner import StepEntry

    _, config, folder, sequences, _, w64 = model_case
    tokens = sequences["s31"]
    _, layers = plain.forward(config, w64, tokens, return_layers=True)
    replay = Replay(folder, dtype, 64)
    replay.cache.open(1)
    replay.cache.manager.ensure(1, len(tokens))
    replay.cache.clear_new_slots()
    ctx = replay.runner._build_context([StepEntry(1, tokens)], [0], [])
    x = replay.model.embedding.forward(ctx)
    for index, call in enumerate(replay.model.schedule):
        replay.model.blocks[call.layer].forward(ctx, replay.runner._view(call, replay.runner._tables), x, None)
        error = np.abs(x.double().cpu().numpy() - layers[index]).max() / np.abs(layers[index]).max()
        assert error <= (1e-5 if dtype == "float32" else 6e-2), f"layer {index} ({config['layers'][index]['type']}): {error:.2e}"
    replay.runner.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_one_after_another_in_a_pool_for_one(model_case, dtype):
    _, _, folder, sequences, expected, _ = model_case
    replay = Replay(folder, dtype, 152, slots=1)
    for key, tokens in sequences.items():
        replay.step([(key, tokens)], end=(key,))
    check_all(replay, sequences, expected, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token(model_case, dtype):
    """All but the last 40 tokens as one portion, the rest one by one (captured steps replayed)."""
    _, _, folder, sequences, expected, _ = model_case
    replay = Replay(folder, dtype, 152, slots=1)
    for key, tokens in sequences.items():
        head = max(0, len(tokens) - 40)
        if head:
            replay.step([(key, tokens[:head])])
        for position in range(head, len(tokens)):
            replay.step([(key, [tokens[position]])], end=(key,) if position == len(tokens) - 1 else ())
    check_all(replay, sequences, expected, dtype, "token by token")
    assert replay.runner.graph_replays > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2,), (3, 1, 2, 8, 1, 17), (7, 9, 64)])
def test_portions_of_changing_size(model_case, dtype, sizes):
    _, _, folder, sequences, expected, _ = model_case
    replay = Replay(folder, dtype, 152, slots=1)
    for key, tokens in sequences.items():
        at, turn = 0, 0
        while at < len(tokens):
            size = min(sizes[turn % len(sizes)], len(tokens) - at)
            replay.step([(key, tokens[at : at + size])], end=(key,) if at + size == len(tokens) else ())
            at, turn = at + size, turn + 1
    check_all(replay, sequences, expected, dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(model_case, dtype):
    """Up to three live requests (three slots, 38 pages of 8 for sequences that need 46 in all): portions
    of some beside single tokens of others, requests left out of steps, and every request that
    ends hands its pages and its slot to one that starts later."""
    _, config, folder, sequences, expected, _ = model_case
    replay = Replay(folder, dtype, 304, slots=3)
    rng = np.random.default_rng(9)
    waiting = ["s150", "s70", "s31", "s9", "s3", "s2", "s1", "again70", "again9"]
    sequences = dict(sequences, again70=sequences["s70"], again9=sequences["s9"])
    expected = dict(expected, again70=expected["s70"], again9=expected["s9"])
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
    check_all(replay, sequences, expected, dtype, "mixed")
    stats = replay.cache.stats()
    assert stats["free_state_slots"] == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_case, dtype):
    """Four tokens of prompt, then 330 single tokens: the recurrent state and the latent cache after
    hundreds of steps, across many pages."""
    _, config, folder, _, _, w64 = model_case
    tokens = [int(t) for t in np.random.default_rng(6).integers(0, config["vocab"], 334)]
    want = plain.forward(config, w64, tokens)
    replay = Replay(folder, dtype, 384, slots=1)
    replay.step([("long", tokens[:4])])
    for token in tokens[4:]:
        replay.step([("long", [token])])
    error = row_error(replay.of("long", len(tokens)), want)
    assert error.max() <= TOLERANCE[dtype], f"position {int(error.argmax())}: {error.max():.2e}"
    assert error.mean() <= MEAN_TOLERANCE[dtype] and error[-50:].mean() <= MEAN_TOLERANCE[dtype], f"mean {error.mean():.2e}, last 50 {error[-50:].mean():.2e}"


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
        assert row_error(got, np.concatenate(want)).max() <= TOLERANCE[dtype]


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
