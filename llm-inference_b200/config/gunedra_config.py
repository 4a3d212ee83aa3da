"""Configuration of the Gunedra design: a list of layers, each with a mixer and a feed-forward.

``config.json`` of this design is nested::

    {"architecture": "Gunedra", "vocab": V, "width": D, "residual_mult": m,
     "embedding": {"scale": s}, "norm": {"eps": e, "groups": G},
     "layers": [{"type": "latent_attention" | "channel_delta", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F} | null}, ...]}

Mixer sizes: ``latent_attention``: ``heads, dim, rot_dim, vdim, kv_rank, scale,
rot: {base, dims}``; ``channel_delta``: ``heads, kv_heads, dim, vdim, conv``. The inner sizes of
the delta rule's two low-rank projection pairs are the checkpoint's tensor shapes; the optional
keys ``decay_rank`` / ``gate_rank`` exist only so that random weights can be drawn from a
configuration alone. The design has no position limit and no end-of-sequence token.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, ClassVar

from .model_config import ConfigError, ModelConfig, _take

MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank"),
    "channel_delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
}


@dataclass(frozen=True)
class GunedraConfig(ModelConfig):
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    norm_eps: float = 0.0
    norm_groups: int = 1
    layers: tuple[dict[str, Any], ...] = field(default_factory=tuple)

    ARCHITECTURE: ClassVar[str] = "Gunedra"
    MODEL_TYPE: ClassVar[str] = "gunedra"

    @classmethod
    def from_json_dict(cls, raw: dict[str, Any]) -> "GunedraConfig":
        def section(name: str) -> dict[str, Any]:
            value = raw.get(name)
            if not isinstance(value, dict):
                raise ConfigError(f"config.json key '{name}' must be an object")
            return value

        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        norm = section("norm")
        config = cls(
            architecture=cls.ARCHITECTURE,
            vocab_size=_take(raw, "vocab", int),
            hidden_size=_take(raw, "width", int),
            num_hidden_layers=len(layers),
            max_position_embeddings=cls.MAX_POSITIONS,
            eos_token_ids=(),
            embedding_scale=_take(section("embedding"), "scale", float),
            residual_mult=_take(raw, "residual_mult", float),
            norm_eps=_take(norm, "eps", float),
            norm_groups=_take(norm, "groups", int),
            layers=tuple(copy.deepcopy(layer) for layer in layers),
        )
        config.validate()
        return config

    def validate(self) -> None:
        super().validate()
        if not (math.isfinite(self.norm_eps) and self.norm_eps > 0):
            raise ConfigError(f"norm.eps={self.norm_eps} must be finite and positive")
        if self.norm_groups <= 0 or self.hidden_size % self.norm_groups:
            raise ConfigError(f"width={self.hidden_size} does not cut into norm.groups={self.norm_groups} equal parts")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_KEYS:
                raise ConfigError(f"{where}.type must be one of {sorted(MIXER_KEYS)}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            for key in MIXER_KEYS[layer["type"]]:
                if _take(mixer, key, int) <= 0:
                    raise ConfigError(f"{where}.mixer.{key} must be positive")
            if layer["type"] == "latent_attention":
                rot = mixer.get("rot")
                if not isinstance(rot, dict):
                    raise ConfigError(f"{where}.mixer.rot must be an object")
                dims = _take(rot, "dims", int)
                if dims % 2 or not 0 <= dims <= mixer["rot_dim"] or _take(rot, "base", float) <= 0:
                    raise ConfigError(f"{where}.mixer.rot: dims must be even and at most rot_dim, base positive")
                _take(mixer, "scale", float)
            elif mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"{where}.mixer: heads={mixer['heads']} is not a multiple of kv_heads={mixer['kv_heads']}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp.kind must be 'dense' (or mlp null)")
                if not 0 < _take(mlp, "ff", int) <= self.MAX_INTERMEDIATE:
                    raise ConfigError(f"{where}.mlp.ff is out of range")

    def to_json_dict(self) -> dict[str, Any]:
        return {
            "architecture": self.architecture,
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "residual_mult": self.residual_mult,
            "embedding": {"scale": self.embedding_scale},
            "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
            "layers": [copy.deepcopy(layer) for layer in self.layers],
        }
