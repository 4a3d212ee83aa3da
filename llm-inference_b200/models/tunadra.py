"""Tunadra as a recipe of parts.

``x = table[token] * scale + e(position)`` (sines and cosines in alternating columns) fills ``n`` residual
streams per token. Each layer is pre-norm over those streams (hyper-connections): a sublayer reads a
learned combination of the streams through an RMS norm and its output goes back into all of them
through a learned ``n x n`` mix plus a learned weight per stream. The mixer is a recurrent one (matrix
state per head, decay per channel, bonus for the current token) or attention without position
encoding (unit-RMS queries and keys, values blended with those of the first such layer, a sigmoid gate
per head); the feed-forward is a routed mixture of clamped gated experts with a shared expert, or
absent. The sum of the streams goes through a last RMS norm and an untied head whose logits are
soft-capped. Every size, constant and the order of the layers come from the configuration.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tunadra_config import TunadraConfig
from ..parts.base import PartSpec
from ..parts.model import ModelRecipe


def tunadra_recipe(config: TunadraConfig) -> ModelRecipe:
    hidden, eps = config.hidden_size, config.norm_eps
    streams = config.streams or 1
    connected = config.streams is not None
    layers = []
    value_source_seen = False
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        sizes = layer["mixer"]
        if layer["type"] == "wkv":
            mixer = PartSpec(
                "wkv",
                dict(prefix=prefix + "mix.", hidden_size=hidden, heads=sizes["heads"], dim=sizes["dim"], eps=eps, decay_rank=sizes.get("decay_rank")),
            )
        else:
            values = None
            if sizes.get("v_mix"):
                values = "blend" if value_source_seen else "publish"
                value_source_seen = True
            mixer = PartSpec(
                "gated_attention",
                dict(
                    prefix=prefix + "mix.", hidden_size=hidden, heads=sizes["heads"], kv_heads=sizes["kv_heads"], dim=sizes["dim"],
                    vdim=sizes["vdim"], scale=sizes["scale"], eps=eps, qk_norm=True, gate=True, values=values,
                    has_blend_tensor=True,  # a checkpoint may carry the factor for a layer that does not blend: it is read past
                ),
            )
        mlp = layer.get("mlp")
        feed_forward = None
        if mlp is not None:
            router, shared = mlp["router"], mlp.get("shared")
            groups = router.get("groups") or {"count": 1, "keep": 1}
            feed_forward = PartSpec(
                "routed_experts",
                dict(
                    prefix=prefix + "mlp.", hidden_size=hidden, experts=router["experts"], top=router["top"],
                    intermediate_size=mlp["expert"]["ff"], limit=mlp["expert"]["limit"], route_scale=router["scale"],
                    group_count=groups["count"], group_keep=groups["keep"],
                    shared_size=shared["ff"] if shared else None, shared_limit=shared["limit"] if shared else None,
                ),
            )

        def norm(q: int) -> PartSpec:
            read = f"{prefix}hc{q}.in" if connected else None
            return PartSpec("streams_rmsnorm", dict(name=f"{prefix}norm{q}", hidden_size=hidden, eps=eps, streams=streams, read=read))

        layers.append(
            PartSpec(
                "hyper_connections",
                dict(
                    mixer=mixer, feed_forward=feed_forward, mixer_norm=norm(1), feed_forward_norm=norm(2) if mlp is not None else None,
                    streams=streams, connections=(prefix + "hc1.", prefix + "hc2.") if connected else None,
                    unused=() if mlp is not None else (prefix + "norm2",),
                ),
            )
        )
    return ModelRecipe(
        config=config,
        embedding=PartSpec(
            "sinusoid_embedding",
            dict(name="embed", vocab_size=config.vocab_size, hidden_size=hidden, scale=config.embedding_scale, streams=streams),
        ),
        layers=layers,
        final_norm=PartSpec("streams_rmsnorm", dict(name="final.norm", hidden_size=hidden, eps=eps, streams=streams)),
        head=PartSpec("linear_head", dict(name="head", suffix="", vocab_size=config.vocab_size, hidden_size=hidden, softcap=config.logit_softcap)),
    )


register_architecture(TunadraConfig.ARCHITECTURE, TunadraConfig.from_json_dict, tunadra_recipe, model_types=(TunadraConfig.MODEL_TYPE,))
