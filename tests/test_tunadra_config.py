"""Tunadra on the CPU: registry, configuration errors, tensor names and shapes, seeded folders, and the
plain implementation against second formulations of its mechanisms."""

from __future__ import annotations

import copy
import json

import numpy as np
import pytest

from plain import tunadra_plain as plain
from tunadra_helpers import ALPHA, BETA, CONFIGS, GAMMA, draw_weights


def parsed(raw):
    from llm_inference_b200 import models  # noqa: F401
    from llm_inference_b200.config.registry import parse_config

    return parse_config(json.loads(json.dumps(raw)))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_configuration_round_trip_and_tensor_names(name):
    from llm_inference_b200.parts.model import Model

    raw = CONFIGS[name]
    entry, config = parsed(raw)
    assert entry.name == "Tunadra" and config.to_json_dict() == raw
    specs = {spec.name: spec for spec in Model(entry.recipe(config)).tensor_specs()}
    weights = draw_weights(raw, 3)
    assert all(specs[n].fits(tuple(t.shape)) for n, t in weights.items())
    assert {n for n, s in specs.items() if not s.optional} <= set(weights) <= set(specs)  # the first mixing layer's own factor is read past
    kinds = {type(s).__name__ for s in Model(entry.recipe(config)).cache_specs().values()}
    assert kinds == {"KVCacheSpec", "StateSpec"}


def test_recipe_reads_every_size_from_the_configuration():
    from llm_inference_b200.parts.model import Model

    entry, config = parsed(BETA)
    model = Model(entry.recipe(config))
    first, second = model.blocks[0], model.blocks[1]
    assert (first.mixer.heads, first.mixer.dim, first.streams) == (1, 6, 4)
    assert (first.feed_forward.experts, first.feed_forward.top, first.feed_forward.group_count, first.feed_forward.group_keep) == (5, 1, 5, 3)
    assert first.feed_forward.shared_size == 0 and first.feed_forward.route_scale == 0.7
    assert (second.mixer.heads, second.mixer.kv_heads, second.mixer.dim, second.mixer.vdim, second.mixer.scale) == (5, 1, 72, 40, 0.35)
    assert second.mixer.row_dim == 128 and model.blocks[3].mixer.row_dim == 144 and second.mixer.values is None
    assert (second.feed_forward.group_count, second.feed_forward.limit) == (1, 0.8)
    assert model.blocks[2].feed_forward is None and model.head.softcap == 7.5 and model.embedding.scale == 0.6
    # the first layer that mixes values gives them, the later ones blend; a layer between them does neither
    alpha = Model(parsed(ALPHA)[0].recipe(parsed(ALPHA)[1]))
    assert [getattr(b.mixer, "values", "-") for b in alpha.blocks] == ["publish", "-", None, "blend", "-"]
    gamma = Model(parsed(GAMMA)[0].recipe(parsed(GAMMA)[1]))
    assert gamma.blocks[0].streams == 1 and gamma.blocks[0].connections is None


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.update(width=47), "even"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c.update(logit_softcap=-1.0), "softcap"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), "agree"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(experts=7), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0.0), "limit"),
    (lambda c: c["layers"][1]["mixer"].update(dim=0), "positive"),
])
def test_configuration_errors(change, message):
    from llm_inference_b200.config.model_config import ConfigError

    raw = copy.deepcopy(ALPHA)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        parsed(raw)


def test_seeded_folder_round_trip(tmp_path):
    from llm_inference_b200.config.model_config import read_config_json
    from llm_inference_b200.weights.loader import load_weights
    from llm_inference_b200.weights.random_init import write_model_folder

    entry, config = parsed(ALPHA)
    folder = write_model_folder(tmp_path / "m", config, seed=5)
    assert read_config_json(folder) == ALPHA
    tensors = load_weights(folder, entry.recipe(config).tensor_specs())
    assert "l0.mix.vmix" not in tensors and tensors["l3.mix.vmix"].shape == () and tensors["l1.mix.w1"].shape == (5, 48) and tensors["l0.hc1.mix"].shape == (2, 2)


# --- the plain implementation against second formulations ----------------------------------------------


def test_plain_sinusoid_is_a_rotation_by_position():
    """sin and cos of (p + d) f follow from those of p f by the angle-sum rule; position 0 gives 0, 1, 0, 1, ..."""
    width = 12
    e = plain.sinusoid(np.arange(40), width)
    assert np.allclose(e[0, 0::2], 0) and np.allclose(e[0, 1::2], 1)
    f = 10000.0 ** (-np.arange(width // 2) * 2.0 / width)
    d = 7
    sin, cos = e[:-d, 0::2], e[:-d, 1::2]
    assert np.allclose(e[d:, 0::2], sin * np.cos(d * f) + cos * np.sin(d * f))
    assert np.allclose(e[d:, 1::2], cos * np.cos(d * f) - sin * np.sin(d * f))


def test_plain_streams_with_identity_weights_are_a_residual_sum():
    rng = np.random.default_rng(0)
    xs, y = rng.normal(size=(3, 5, 8)), rng.normal(size=(5, 8))
    new = plain.streams_write(xs, y, np.eye(3), np.ones(3))
    assert np.allclose(new, xs + y[None])
    assert np.allclose(plain.streams_read(new, np.ones(3)), xs.sum(axis=0) + 3 * y)
    # the mix is indexed [from, to]
    mix = np.zeros((3, 3))
    mix[0, 2] = 1.0
    assert np.allclose(plain.streams_write(xs, y, mix, np.zeros(3))[2], xs[0]) and np.allclose(plain.streams_write(xs, y, mix, np.zeros(3))[0], 0)


def test_plain_recurrence_equals_its_unrolled_sum():
    """o_t = sum_{j<t} (r_t . (prod_{j<m<t} w_m) k_j) v_j + (r_t . u k_t) v_t, head by head."""
    rng = np.random.default_rng(1)
    width, heads, dim, tokens = 10, 2, 3, 6
    w = {"m." + n: rng.normal(0, 0.5, (heads * dim, width)) for n in "rkvg"}
    w.update({"m.mu." + n: rng.uniform(0, 1, width) for n in "rkvgw"})
    w.update({"m.w1": rng.normal(0, 0.5, (4, width)), "m.w2": rng.normal(0, 0.5, (heads * dim, 4)), "m.w0": rng.normal(-1, 1, heads * dim),
              "m.u": rng.normal(0, 1, (heads, dim)), "m.norm": np.ones(heads * dim), "m.o": np.eye(heads * dim)})
    w["m.g"][:] = 0
    h = rng.normal(size=(tokens, width))
    out, (last, state) = plain.wkv_mixer(h, w, "m.", heads, dim, 1e-9)
    assert np.allclose(last, h[-1])
    shifted = np.vstack([np.zeros(width), h[:-1]])
    blend = {n: h + (shifted - h) * w["m.mu." + n] for n in "rkvgw"}
    r, k, v = ((blend[n] @ w["m." + n].T).reshape(tokens, heads, dim) for n in "rkv")
    decay = np.exp(-np.exp(np.tanh(blend["w"] @ w["m.w1"].T) @ w["m.w2"].T + w["m.w0"])).reshape(tokens, heads, dim)
    for n in range(heads):
        for t in range(tokens):
            o = (r[t, n] * w["m.u"][n] * k[t, n]).sum() * v[t, n]
            for j in range(t):
                carried = k[j, n] * np.prod(decay[j + 1 : t, n], axis=0)
                o = o + (r[t, n] * carried).sum() * v[j, n]
            want = o / np.sqrt((o * o).mean() + 1e-9) * 0.0  # the gate is silu(0) = 0
            assert np.allclose(out[t, n * dim : (n + 1) * dim], want)
    # with an open gate the read-out itself shows: g = large -> silu(g) ~ g
    w["m.g"][:] = 0
    assert state.shape == (heads, dim, dim)
    unrolled = sum(np.outer(k[j, 0] * np.prod(decay[j + 1 :, 0], axis=0), v[j, 0]) for j in range(tokens))
    assert np.allclose(state[0], unrolled)


def test_plain_attention_equals_a_masked_softmax_and_is_cut_anywhere():
    rng = np.random.default_rng(2)
    sizes = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.9}
    width, tokens = 24, 9
    w = {"a.q": rng.normal(size=(24, width)), "a.k": rng.normal(size=(12, width)), "a.v": rng.normal(size=(10, width)),
         "a.g": rng.normal(size=(4, width)), "a.o": rng.normal(size=(width, 20)), "a.vmix": np.asarray(0.3)}
    h = rng.normal(size=(tokens, width))
    whole, cache, raw = plain.attention_mixer(h, w, "a.", sizes, 1e-6)
    q, k, v, gate = plain.attention_project(h, w, "a.", 4, 2, 6, 5, 1e-6)
    assert np.allclose((q * q).mean(axis=-1), 1, atol=1e-4) and np.allclose(raw, v)
    for n in range(4):
        scores = q[:, n] @ k[:, n // 2].T * 0.9
        scores[np.triu_indices(tokens, 1)] = -np.inf
        p = np.exp(scores - scores.max(axis=1, keepdims=True))
        o = (p / p.sum(axis=1, keepdims=True)) @ v[:, n // 2] * gate[:, n : n + 1]
        assert np.allclose((whole @ np.linalg.pinv(w["a.o"].T))[:, n * 5 : (n + 1) * 5], o, atol=1e-8)
    first, cache, _ = plain.attention_mixer(h[:4], w, "a.", sizes, 1e-6)
    rest, _, _ = plain.attention_mixer(h[4:], w, "a.", sizes, 1e-6, 4, cache)
    assert np.allclose(np.vstack([first, rest]), whole)
    other = rng.normal(size=(tokens, 2, 5))
    blended, (_, values), _ = plain.attention_mixer(h, w, "a.", sizes, 1e-6, 0, None, other, True)
    assert np.allclose(values, 0.7 * v + 0.3 * other) and not np.allclose(blended, whole)


def test_plain_router_against_a_search_over_all_choices():
    rng = np.random.default_rng(3)
    for experts, groups, keep, top in [(8, 4, 2, 3), (6, 2, 1, 2), (9, 3, 2, 4), (5, 5, 2, 2), (4, 1, 1, 4)]:
        size = experts // groups
        for _ in range(30):
            s = rng.uniform(0, 1, experts)
            group_score = [np.sort(s[g * size : (g + 1) * size])[-2:].sum() for g in range(groups)]
            kept = sorted(range(groups), key=lambda g: -group_score[g])[:keep]
            allowed = [e for e in range(experts) if e // size in kept]
            want = sorted(allowed, key=lambda e: -s[e])[:top]
            assert sorted(plain.route(s, top, groups, keep)) == sorted(want)


def test_plain_expert_clamps_and_mixture_weights():
    rng = np.random.default_rng(4)
    width, ff = 6, 4
    w = {"e.gate": rng.normal(size=(ff, width)) * 3, "e.up": rng.normal(size=(ff, width)) * 3, "e.down": np.eye(width, ff)}
    h = rng.normal(size=(5, width))
    g, u = np.minimum(h @ w["e.gate"].T, 1.0), np.clip(h @ w["e.up"].T, -1.0, 1.0)
    assert np.allclose(plain.clamped_expert(h, w, "e.", 1.0)[:, :ff], g / (1 + np.exp(-1.702 * g)) * (u + 1))
    assert (h @ w["e.gate"].T).max() > 1.0 and (h @ w["e.up"].T).min() < -1.0
    # two experts, both chosen: weights are the scores over their sum, times the scale; a shared expert is added unweighted
    mlp = {"expert": {"ff": ff, "limit": 50.0}, "router": {"experts": 2, "top": 2, "scale": 3.0}, "shared": {"ff": ff, "limit": 50.0}}
    w = {f"m.{e}.{n}": rng.normal(size=(ff, width) if n != "down" else (width, ff)) for e in ("e0", "e1", "shared") for n in ("gate", "up", "down")}
    w["m.router"] = rng.normal(size=(2, width))
    s = plain.sigmoid(h @ w["m.router"].T)
    want = sum((s[:, e : e + 1] / s.sum(axis=1, keepdims=True) * 3.0) * plain.clamped_expert(h, w, f"m.e{e}.", 50.0) for e in range(2))
    assert np.allclose(plain.moe(h, w, "m.", mlp), want + plain.clamped_expert(h, w, "m.shared.", 50.0))
