"""Gunedra as a recipe of parts.

``x = table[token] * scale``. Each layer adds the grouped RMS norm of its branches' outputs, times a
learned per-column scale and a constant, to a 32-bit stream that the branches read directly:
``x += m * ls1 * norm1(mixer(x)); x += m * ls2 * norm2(ff(x))``; what a layer hands on is a learned
weighted average of the embedding's output and all layers' results so far. The mixer is attention
over cached low-rank latents (interleaved rotary part, sink in the softmax, a gate per head) or a
gated delta rule with a decay per key channel; the feed-forward is ``down(PolyNorm(up(x)))`` or
absent. A last grouped norm, then logits against the embedding table itself (without its scale).
Every size, constant and the order of the layers come from the configuration.
"""

from __future__ import annotations

from ..config.gunedra_config import GunedraConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from ..parts.model import ModelRecipe


def gunedra_recipe(config: GunedraConfig) -> ModelRecipe:
    hidden, eps, groups = config.hidden_size, config.norm_eps, config.norm_groups
    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        sizes = layer["mixer"]
        if layer["type"] == "latent_attention":
            mixer = PartSpec(
                "latent_attention",
                dict(
                    prefix=prefix + "mix.", hidden_size=hidden, heads=sizes["heads"], dim=sizes["dim"], rot_dim=sizes["rot_dim"],
                    vdim=sizes["vdim"], rank=sizes["kv_rank"], scale=sizes["scale"], eps=eps,
                    position=PartSpec(
                        "rotary",
                        dict(head_dim=sizes["rot_dim"], theta=sizes["rot"]["base"], rotary_dims=sizes["rot"]["dims"], interleaved=True),
                    ),
                ),
            )
        else:
            mixer = PartSpec(
                "channel_delta",
                dict(
                    prefix=prefix + "mix.", hidden_size=hidden, heads=sizes["heads"], kv_heads=sizes["kv_heads"], dim=sizes["dim"],
                    vdim=sizes["vdim"], taps=sizes["conv"], eps=eps, decay_rank=sizes.get("decay_rank"), gate_rank=sizes.get("gate_rank"),
                ),
            )
        mlp = layer.get("mlp")
        feed_forward = None
        if mlp is not None:
            feed_forward = PartSpec("poly_norm", dict(prefix=prefix + "mlp.", hidden_size=hidden, intermediate_size=mlp["ff"], eps=eps))

        def norm(name: str) -> PartSpec:
            return PartSpec("grouped_rmsnorm", dict(name=name, hidden_size=hidden, groups=groups, eps=eps))

        layers.append(
            PartSpec(
                "post_norm_residual",
                dict(
                    mixer=mixer, feed_forward=feed_forward, mixer_norm=norm(prefix + "norm1"),
                    feed_forward_norm=norm(prefix + "norm2") if mlp is not None else None, hidden_size=hidden,
                    mult=config.residual_mult, mixer_scale=prefix + "ls1", feed_forward_scale=prefix + "ls2",
                    depth_mix=dict(tensor=prefix + "dwa", index=index, layers=len(config.layers)),
                    unused=() if mlp is not None else (prefix + "norm2", prefix + "ls2"),
                ),
            )
        )
    return ModelRecipe(
        config=config,
        embedding=PartSpec(
            "token_embedding",
            dict(name="embed", suffix="", vocab_size=config.vocab_size, hidden_size=hidden, scale=config.embedding_scale, cast=True),
        ),
        layers=layers,
        final_norm=PartSpec("grouped_rmsnorm", dict(name="final.norm", hidden_size=hidden, groups=groups, eps=eps)),
        head=PartSpec("linear_head", dict(name="lm_head", suffix="", vocab_size=config.vocab_size, hidden_size=hidden, tied_to="embed")),
    )


register_architecture(GunedraConfig.ARCHITECTURE, GunedraConfig.from_json_dict, gunedra_recipe, model_types=(GunedraConfig.MODEL_TYPE,))
