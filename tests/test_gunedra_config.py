"""Gunedra without a GPU: the configuration reader, the registry, tensor names, the loader's open
sizes, and the plain implementation's mechanisms against second formulations of the same maths."""

from __future__ import annotations

import json

import numpy as np
import pytest
import torch

from gunedra_helpers import ALPHA, BETA, as_float64, draw_weights, write_folder
from plain import gunedra_plain as plain


def test_registry_reads_the_architecture_from_a_plain_string_and_round_trips():
    from llm_inference_b200 import models  # noqa: F401
    from llm_inference_b200.config import GunedraConfig, parse_config

    entry, config = parse_config(json.loads(json.dumps(BETA)))
    assert entry.name == "Gunedra" and isinstance(config, GunedraConfig)
    assert (config.vocab_size, config.hidden_size, config.num_hidden_layers) == (131, 40, 3)
    assert (config.norm_groups, config.norm_eps, config.residual_mult, config.embedding_scale) == (1, 3e-4, 1.3, 0.7)
    assert config.eos_token_ids == () and config.max_position_embeddings >= 1 << 20
    assert parse_config(config.to_json_dict())[1] == config


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="other"), "type"),
    (lambda c: c["norm"].update(groups=3), "groups"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=2), "kv_heads"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c.pop("embedding"), "embedding"),
])
def test_bad_configurations_are_refused(change, message):
    from llm_inference_b200 import models  # noqa: F401
    from llm_inference_b200.config import ConfigError, parse_config

    raw = json.loads(json.dumps(BETA))
    change(raw)
    with pytest.raises(ConfigError, match=message):
        parse_config(raw)


def test_the_recipe_asks_for_exactly_the_tensors_of_the_design(tmp_path):
    from llm_inference_b200 import models  # noqa: F401
    from llm_inference_b200.config import parse_config
    from llm_inference_b200.weights import WeightsError, load_weights

    for config in (ALPHA, BETA):
        entry, parsed = parse_config(config)
        specs = entry.recipe(parsed).tensor_specs()
        weights = draw_weights(config, 1)
        required = {s.name: s for s in specs if not s.optional}
        assert set(required) == set(weights)
        for name, spec in required.items():
            assert spec.fits(tuple(weights[name].shape)), name
    # inner sizes that only the checkpoint knows: the configuration need not name them ...
    bare = json.loads(json.dumps(ALPHA))
    for layer in bare["layers"]:
        layer["mixer"].pop("decay_rank", None), layer["mixer"].pop("gate_rank", None)
    entry, parsed = parse_config(bare)
    folder = write_folder(tmp_path / "m", bare, draw_weights(ALPHA, 1))
    loaded = load_weights(folder, entry.recipe(parsed).tensor_specs())
    assert loaded["l1.mix.a1"].shape == (5, 48) and loaded["l3.mix.g2"].shape == (16, 2)
    # a layer without a feed-forward may still carry its second norm and scale: they are read past
    extra = dict(draw_weights(ALPHA, 1), **{"l2.norm2": torch.ones(48, dtype=torch.bfloat16), "l2.ls2": torch.ones(48, dtype=torch.bfloat16)})
    load_weights(write_folder(tmp_path / "x", bare, extra), entry.recipe(parsed).tensor_specs())
    # ... and every other mismatch is still named
    broken = draw_weights(ALPHA, 1)
    broken["l0.mix.sink"] = broken["l0.mix.sink"][:2]
    del broken["l2.dwa"]
    with pytest.raises(WeightsError) as error:
        load_weights(write_folder(tmp_path / "b", bare, broken), entry.recipe(parsed).tensor_specs())
    assert error.value.missing == ["l2.dwa"] and [w[0] for w in error.value.wrong_shape] == ["l0.mix.sink"]


def test_a_seeded_model_folder_can_be_drawn_when_the_configuration_names_the_inner_sizes(tmp_path):
    from llm_inference_b200 import models  # noqa: F401
    from llm_inference_b200.config import parse_config
    from llm_inference_b200.weights import load_weights, write_model_folder

    entry, parsed = parse_config(ALPHA)
    folder = write_model_folder(tmp_path / "drawn", parsed, seed=3)
    tensors = load_weights(folder, entry.recipe(parsed).tensor_specs())
    assert tensors["l1.mix.a2"].shape == (32, 5) and tensors["l3.dwa"].shape == (5,)
    bare = json.loads(json.dumps(ALPHA))
    bare["layers"][1]["mixer"].pop("decay_rank")
    with pytest.raises(ValueError, match="only a checkpoint gives"):
        write_model_folder(tmp_path / "bare", parse_config(bare)[1], seed=3)


# --- the plain implementation against second formulations -------------------------------------------------


def test_plain_rotation_keeps_lengths_and_depends_on_distance_only():
    rng = np.random.default_rng(0)
    a, b = rng.normal(size=(1, 12)), rng.normal(size=(1, 12))
    for dims in (12, 8):
        ra, rb = plain.rotate_interleaved(a, [7], 300.0, dims), plain.rotate_interleaved(b, [3], 300.0, dims)
        sa, sb = plain.rotate_interleaved(a, [104], 300.0, dims), plain.rotate_interleaved(b, [100], 300.0, dims)
        assert np.allclose(np.linalg.norm(ra), np.linalg.norm(a))
        assert np.allclose(ra @ rb.T, sa @ sb.T)
        assert np.array_equal(ra[:, dims:], a[:, dims:])
    one = plain.rotate_interleaved(np.array([[1.0, 0.0, 1.0, 0.0]]), [2], 100.0, 4)
    assert np.allclose(one, [[np.cos(2.0), np.sin(2.0), np.cos(0.2), np.sin(0.2)]])


def test_plain_sink_attention_is_a_softmax_over_the_keys_and_one_extra_logit():
    rng = np.random.default_rng(1)
    q, k, v = rng.normal(size=(5, 2, 6)), rng.normal(size=(5, 2, 6)), rng.normal(size=(5, 2, 3))
    sink = np.array([0.5, -1.0])
    got = plain.sink_softmax_attention(q, k, v, sink, 0.4)
    for h in range(2):
        for i in range(5):
            logits = np.concatenate([[sink[h]], 0.4 * (k[: i + 1, h] @ q[i, h])])
            p = np.exp(logits) / np.exp(logits).sum()
            assert np.allclose(got[i, h], p[1:] @ v[: i + 1, h])


def test_plain_delta_rule_equals_its_column_form_and_convolution_equals_numpy():
    rng = np.random.default_rng(2)
    t, dk, dv = 9, 5, 4
    q, k, v = rng.normal(size=(t, dk)), rng.normal(size=(t, dk)), rng.normal(size=(t, dv))
    beta, decay = rng.uniform(0.2, 0.9, t), rng.uniform(0.3, 1.0, (t, dk))
    got = plain.gated_delta_rule(q, k, v, beta, decay)
    for col in range(dv):  # the columns of the state never mix
        s = np.zeros(dk)
        for i in range(t):
            s = decay[i] * s
            s = s + k[i] * beta[i] * (v[i, col] - s @ k[i])
            assert np.isclose(got[i, col], s @ q[i])
    x, taps = rng.normal(size=(11, 3)), rng.normal(size=(3, 4))
    y = plain.short_convolution(x, taps)
    for c in range(3):
        pre = np.convolve(x[:, c], taps[c, ::-1])[:11]
        assert np.allclose(y[:, c], pre / (1 + np.exp(-pre)))


def test_plain_forward_of_a_prefix_is_the_prefix_of_the_forward():
    weights = as_float64(draw_weights(ALPHA, 2))
    tokens = [int(t) for t in np.random.default_rng(3).integers(0, ALPHA["vocab"], 20)]
    whole = plain.forward(ALPHA, weights, tokens)
    assert np.allclose(plain.forward(ALPHA, weights, tokens[:13]), whole[:13])
    assert whole.shape == (20, ALPHA["vocab"]) and np.isfinite(whole).all() and whole.std() > 0.1
