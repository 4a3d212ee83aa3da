"""Configuration of the Tunadra design: a list of layers, each a mixer plus an optional routed feed-forward.

``config.json`` of this design is nested::

    {"architecture": "Tunadra", "vocab": V, "width": D, "streams": n, "logit_softcap": c,
     "embedding": {"scale": s}, "norm": {"eps": e},
     "layers": [{"type": "wkv" | "attention", "mixer": {...}, "mlp": {...} | null}, ...]}

Mixer sizes: ``wkv``: ``heads, dim`` (the inner size of its low-rank decay pair is the checkpoint's;
the optional key ``decay_rank`` exists only so that random weights can be drawn from a configuration
alone); ``attention``: ``heads, kv_heads, dim, vdim, scale`` and optionally ``v_mix``.
Feed-forward: ``{"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top", "scale",
"groups": {"count", "keep"}}, "shared": {"ff", "limit"}}``; ``groups`` and ``shared`` may be absent
(one group; no shared expert). Without ``streams`` a layer adds its branches to one residual stream.
The design has no position limit and no end-of-sequence token.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, ClassVar

from .model_config import ConfigError, ModelConfig, _take

MIXER_KEYS = {
    "wkv": ("heads", "dim"),
    "attention": ("heads", "kv_heads", "dim", "vdim"),
}


@dataclass(frozen=True)
class TunadraConfig(ModelConfig):
    embedding_scale: float = 1.0
    norm_eps: float = 0.0
    streams: int | None = None  # None: one residual stream without hyper-connection tensors
    logit_softcap: float | None = None
    layers: tuple[dict[str, Any], ...] = field(default_factory=tuple)

    ARCHITECTURE: ClassVar[str] = "Tunadra"
    MODEL_TYPE: ClassVar[str] = "tunadra"
    MAX_STREAMS: ClassVar[int] = 8

    @classmethod
    def from_json_dict(cls, raw: dict[str, Any]) -> "TunadraConfig":
        def section(name: str) -> dict[str, Any]:
            value = raw.get(name)
            if not isinstance(value, dict):
                raise ConfigError(f"config.json key '{name}' must be an object")
            return value

        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        config = cls(
            architecture=cls.ARCHITECTURE,
            vocab_size=_take(raw, "vocab", int),
            hidden_size=_take(raw, "width", int),
            num_hidden_layers=len(layers),
            max_position_embeddings=cls.MAX_POSITIONS,
            eos_token_ids=(),
            embedding_scale=_take(section("embedding"), "scale", float),
            norm_eps=_take(section("norm"), "eps", float),
            streams=_take(raw, "streams", int, None),
            logit_softcap=_take(raw, "logit_softcap", float, None),
            layers=tuple(copy.deepcopy(layer) for layer in layers),
        )
        config.validate()
        return config

    def validate(self) -> None:
        super().validate()
        if self.hidden_size % 2:
            raise ConfigError(f"width={self.hidden_size} must be even (sine and cosine columns alternate)")
        if not (math.isfinite(self.norm_eps) and self.norm_eps > 0):
            raise ConfigError(f"norm.eps={self.norm_eps} must be finite and positive")
        if self.streams is not None and not 0 < self.streams <= self.MAX_STREAMS:
            raise ConfigError(f"streams={self.streams} is outside (0, {self.MAX_STREAMS}]")
        if self.logit_softcap is not None and not (math.isfinite(self.logit_softcap) and self.logit_softcap > 0):
            raise ConfigError(f"logit_softcap={self.logit_softcap} must be finite and positive")
        mixed_values = None
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
            if layer["type"] == "attention":
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"{where}.mixer: heads={mixer['heads']} is not a multiple of kv_heads={mixer['kv_heads']}")
                _take(mixer, "scale", float)
                if _take(mixer, "v_mix", bool, False):
                    shape = (mixer["kv_heads"], mixer["vdim"])
                    if mixed_values is not None and mixed_values != shape:
                        raise ConfigError(f"{where}.mixer: layers that mix values must agree on kv_heads and vdim")
                    mixed_values = shape
            mlp = layer.get("mlp")
            if mlp is not None:
                self._validate_mlp(mlp, where + ".mlp")

    def _validate_mlp(self, mlp: Any, where: str) -> None:
        if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
            raise ConfigError(f"{where}.kind must be 'moe' (or mlp null)")
        for name in ("expert", "shared"):
            part = mlp.get(name)
            if part is None and name == "shared":
                continue
            if not isinstance(part, dict):
                raise ConfigError(f"{where}.{name} must be an object")
            if not 0 < _take(part, "ff", int) <= self.MAX_INTERMEDIATE:
                raise ConfigError(f"{where}.{name}.ff is out of range")
            if not _take(part, "limit", float) > 0:
                raise ConfigError(f"{where}.{name}.limit must be positive")
        router = mlp.get("router")
        if not isinstance(router, dict):
            raise ConfigError(f"{where}.router must be an object")
        experts, top = _take(router, "experts", int), _take(router, "top", int)
        _take(router, "scale", float)
        count, keep = 1, 1
        groups = router.get("groups")
        if groups is not None:
            if not isinstance(groups, dict):
                raise ConfigError(f"{where}.router.groups must be an object")
            count, keep = _take(groups, "count", int), _take(groups, "keep", int)
        if experts <= 0 or count <= 0 or experts % count or not 0 < keep <= count:
            raise ConfigError(f"{where}.router: {experts} experts do not form {count} equal groups of which {keep} are kept")
        if not 0 < top <= keep * (experts // count):
            raise ConfigError(f"{where}.router.top={top} does not fit the kept groups")

    def to_json_dict(self) -> dict[str, Any]:
        out = {
            "architecture": self.architecture,
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "embedding": {"scale": self.embedding_scale},
            "norm": {"eps": self.norm_eps},
            "layers": [copy.deepcopy(layer) for layer in self.layers],
        }
        if self.streams is not None:
            out["streams"] = self.streams
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out
