"""Small Tunadra configurations and weights drawn here (not by the engine)."""

from __future__ import annotations

import numpy as np
import torch


def wkv_layer(heads=4, dim=8, decay_rank=5):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": decay_rank}}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, scale=1.2, v_mix=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if v_mix is not None:
        mixer["v_mix"] = v_mix
    return {"type": "attention", "mixer": mixer}


def moe(experts=8, top=2, ff=24, limit=2.0, scale=1.5, groups=(4, 2), shared=(40, 1.5)):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    return mlp


def with_mlp(layer: dict, mlp: dict | None) -> dict:
    return dict(layer, mlp=mlp)


def config_of(width, vocab, layers, streams=3, embedding_scale=2.0, eps=1e-5, softcap=20.0) -> dict:
    out = {"architecture": "Tunadra", "vocab": vocab, "width": width, "embedding": {"scale": embedding_scale}, "norm": {"eps": eps},
           "logit_softcap": softcap, "layers": layers}
    if streams is not None:
        out["streams"] = streams
    return out


# Three configurations that differ in every size. ALPHA: attention first, a layer that mixes values
# after one that does not, a layer without a feed-forward, two streams. BETA: the recurrent layer
# first, one head of a width that is no multiple of four, all query heads on one key/value head, keys
# wider than values and the other way round, one expert per token, groups of one expert, no shared
# expert, four streams. GAMMA: no streams key at all (one residual stream), no groups, every
# attention layer mixing values, heads of 64 (the tensor-core attention kernels' size).
ALPHA = config_of(
    48, 97,
    [
        with_mlp(attention_layer(v_mix=True), moe()),
        with_mlp(wkv_layer(), moe(experts=6, top=3, ff=20, groups=(2, 1), shared=(12, 3.0))),
        with_mlp(attention_layer(heads=2, kv_heads=2, dim=8, vdim=8, scale=2.0), None),
        with_mlp(attention_layer(heads=6, kv_heads=2, dim=24, vdim=24, scale=0.9, v_mix=True), moe(experts=4, top=4, ff=36, groups=(1, 1))),
        with_mlp(wkv_layer(heads=2, dim=40, decay_rank=3), None),
    ],
    streams=2,
)
BETA = config_of(
    40, 131,
    [
        with_mlp(wkv_layer(heads=1, dim=6, decay_rank=2), moe(experts=5, top=1, ff=70, groups=(5, 3), shared=None, scale=0.7)),
        with_mlp(attention_layer(heads=5, kv_heads=1, dim=72, vdim=40, scale=0.35), moe(experts=3, top=2, ff=33, groups=None, limit=0.8)),
        with_mlp(wkv_layer(heads=3, dim=20, decay_rank=7), None),
        with_mlp(attention_layer(heads=3, kv_heads=3, dim=8, vdim=136, scale=3.0), None),
    ],
    streams=4, embedding_scale=0.6, eps=3e-4, softcap=7.5,
)
GAMMA = config_of(
    64, 113,
    [
        with_mlp(attention_layer(heads=3, kv_heads=1, dim=64, vdim=64, scale=0.4, v_mix=True), moe(experts=12, top=3, ff=32, groups=(3, 2), shared=(64, 2.5))),
        with_mlp(wkv_layer(heads=2, dim=32, decay_rank=8), moe(experts=8, top=3, ff=48, groups=None)),
        with_mlp(attention_layer(heads=3, kv_heads=1, dim=64, vdim=64, scale=0.5, v_mix=True), moe(experts=2, top=1, ff=16, groups=(2, 2))),
    ],
    streams=None, embedding_scale=4.0, softcap=50.0,
)
CONFIGS = {"alpha": ALPHA, "beta": BETA, "gamma": GAMMA}


def draw_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 weights at the scales of a trained model, by tensor name: linear weights N(0, 1/in),
    decays spread between channels that forget in a few tokens and channels that keep hundreds, stream
    weights around a residual connection, router logits wide enough that choices are clear."""
    rng = np.random.default_rng(seed)
    width, vocab = config["width"], config["vocab"]
    n = config.get("streams")
    out: dict[str, np.ndarray] = {}

    def linear(name, rows, cols, gain=1.0):
        out[name] = rng.normal(0.0, gain / np.sqrt(cols), (rows, cols))

    def near_one(name, count, spread=0.2):
        out[name] = 1.0 + rng.normal(0.0, spread, count)

    out["embed"] = rng.normal(0.0, 1.0, (vocab, width))
    linear("head", vocab, width, 2.0)
    near_one("final.norm", width)
    for index, layer in enumerate(config["layers"]):
        p, m = f"l{index}.", layer["mixer"]
        near_one(p + "norm1", width)
        sublayers = 2 if layer.get("mlp") is not None else 1
        if n is not None:
            for q in range(1, sublayers + 1):
                out[f"{p}hc{q}.in"] = rng.normal(1.0 / n, 0.3, n)
                out[f"{p}hc{q}.out"] = rng.normal(0.8, 0.4, n)
                out[f"{p}hc{q}.mix"] = np.eye(n) + rng.normal(0.0, 0.25, (n, n))
        if layer["type"] == "wkv":
            heads, dim = m["heads"], m["dim"]
            inner = heads * dim
            for s in "rkvgw":
                out[p + "mix.mu." + s] = rng.uniform(0.0, 1.0, width)
            for s in "rkv":
                linear(p + "mix." + s, inner, width)
            linear(p + "mix.g", inner, width, 2.0)
            linear(p + "mix.w1", m["decay_rank"], width), linear(p + "mix.w2", inner, m["decay_rank"], 2.0)
            out[p + "mix.w0"] = rng.permutation(np.linspace(-6.0, 0.5, inner))
            out[p + "mix.u"] = rng.normal(0.5, 0.5, (heads, dim))
            near_one(p + "mix.norm", inner)
            linear(p + "mix.o", width, inner)
        else:
            heads, kvh, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            linear(p + "mix.q", heads * dim, width), linear(p + "mix.k", kvh * dim, width), linear(p + "mix.v", kvh * vdim, width)
            linear(p + "mix.g", heads, width, 2.0), linear(p + "mix.o", width, heads * vdim)
            if m.get("v_mix"):
                out[p + "mix.vmix"] = np.asarray(rng.uniform(0.25, 0.6))
        mlp = layer.get("mlp")
        if mlp is not None:
            near_one(p + "norm2", width)
            experts, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            linear(p + "mlp.router", experts, width, 3.0)
            for e in range(experts):
                linear(f"{p}mlp.e{e}.gate", ff, width, 2.0), linear(f"{p}mlp.e{e}.up", ff, width, 2.0), linear(f"{p}mlp.e{e}.down", width, ff)
            if mlp.get("shared"):
                s = mlp["shared"]["ff"]
                linear(p + "mlp.shared.gate", s, width, 2.0), linear(p + "mlp.shared.up", s, width, 2.0), linear(p + "mlp.shared.down", width, s)
    return {name: torch.from_numpy(value if value.ndim == 0 else np.ascontiguousarray(value)).to(torch.bfloat16) for name, value in out.items()}
