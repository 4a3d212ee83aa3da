"""Layers over several residual streams per token (hyper-connections), and the norm that reads them."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import Part, PartSpec, build_part, register_part
from .context import CacheView, StepContext


class StreamsRMSNorm(Part):
    """``y = u / sqrt(mean(u^2) + eps) * weight`` with ``u = sum_s a[s] x_s`` over the token's ``streams``
    residual streams (``x`` is ``[tokens, streams * hidden]``, 32-bit); all 32-bit. ``read`` names the tensor
    that holds ``a``; without it ``u`` is the plain sum (the model's last norm; with one stream, the
    stream itself). A pending branch output (:class:`ops.PendingBranch`) is written into the streams by
    the same kernel first."""

    foldable = False

    def __init__(self, *, name: str, hidden_size: int, eps: float, streams: int = 1, read: str | None = None) -> None:
        self.name, self.hidden_size, self.eps, self.streams, self.read = name, hidden_size, float(eps), int(streams), read
        self.weight: torch.Tensor | None = None
        self.read_weights: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        specs = [TensorSpec(self.name, (self.hidden_size,), init="one_plus_normal")]
        if self.read:
            specs.append(TensorSpec(self.read, (self.streams,), init="half_plus_normal"))
        return specs

    def load(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name].to(device=device, dtype=torch.float32).contiguous()
        if self.read:
            self.read_weights = tensors[self.read].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * 4

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, rows: torch.Tensor | None = None, out_name: str = "normed",
                folded_ok: bool = False) -> torch.Tensor:
        if delta is not None and not isinstance(delta, ops.PendingBranch):
            raise ValueError("a norm over streams takes a pending branch output with its mixing weights")
        count = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer(out_name, (count, self.hidden_size), per_token=rows is None)
        return ops.hyper_norm(ctx, x, delta, self.read_weights, self.weight, self.streams, self.eps, out, rows)


class HyperConnectionBlock(Part):
    """A pre-norm layer over ``streams`` residual streams. For each sublayer (mixer, then feed-forward if
    the layer has one) with its three small tensors ``in [n]``, ``mix [n, n]`` (indexed ``[from, to]``) and
    ``out [n]``: ``u = sum_s in[s] x_s``; ``y = sublayer(norm(u))``; then, all streams at once from the old
    ones, ``x_t <- sum_s mix[s, t] x_s + out[t] y``. Without ``connections`` (tensor-name prefixes of the
    two sublayers) there is one stream and ``x <- x + y``.

    The write of a sublayer's output runs inside the norm kernel that reads the streams next, so the
    block takes the pending output of the layer in front and hands on its own."""

    def __init__(self, *, mixer: PartSpec, feed_forward: PartSpec | None, mixer_norm: PartSpec, feed_forward_norm: PartSpec | None,
                 streams: int = 1, connections: tuple[str, str] | None = None, unused: tuple[str, ...] = ()) -> None:
        self.streams = int(streams)
        self.unused = tuple(unused)  # per-column tensors a checkpoint may carry for a sublayer the layer does not have
        if connections is None and self.streams != 1:
            raise ValueError("several streams need their connection tensors")
        self.mixer_norm = build_part("norm", mixer_norm)
        self.mixer = build_part("mixer", mixer)
        self.feed_forward = build_part("feed_forward", feed_forward) if feed_forward is not None else None
        self.feed_forward_norm = build_part("norm", feed_forward_norm) if feed_forward is not None else None
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None)
        self.graph_safe = all(p.graph_safe for p in self.parts)
        self.connections = tuple(connections) if connections else None
        self.write_weights: list[tuple[torch.Tensor, torch.Tensor] | None] = [None, None]

    def _sublayers(self) -> int:
        return 2 if self.feed_forward is not None else 1

    def tensor_specs(self):
        specs = [spec for part in self.parts for spec in part.tensor_specs()]
        n = self.streams
        for q, prefix in enumerate(self.connections or ()):
            optional = q >= self._sublayers()  # a checkpoint may carry the second sublayer's tensors although the layer has none
            specs.append(TensorSpec(prefix + "mix", (n, n), init="half_plus_normal", optional=optional))
            specs.append(TensorSpec(prefix + "out", (n,), init="half_plus_normal", optional=optional))
            if optional:
                specs.append(TensorSpec(prefix + "in", (n,), init="half_plus_normal", optional=True))
        hidden = self.mixer_norm.hidden_size
        specs += [TensorSpec(name, (hidden,), init="one_plus_normal", optional=True) for name in self.unused]
        return specs

    def load(self, tensors, dtype, device) -> None:
        for part in self.parts:
            part.load(tensors, dtype, device)
        for q in range(self._sublayers()):
            if self.connections:
                prefix = self.connections[q]
                mix = tensors[prefix + "mix"].to(device=device, dtype=torch.float32).contiguous()
                out = tensors[prefix + "out"].to(device=device, dtype=torch.float32).contiguous()
            else:
                mix, out = torch.ones((1, 1), dtype=torch.float32, device=device), torch.ones((1,), dtype=torch.float32, device=device)
            self.write_weights[q] = (mix, out)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part in self.parts)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx: StepContext, cache: CacheView | None, x: torch.Tensor, delta):
        h = self.mixer_norm.forward(ctx, x, delta)
        y = self.mixer.forward(ctx, cache, h)
        pending = ops.PendingBranch(y, *self.write_weights[0])
        if self.feed_forward is None:
            return pending
        h = self.feed_forward_norm.forward(ctx, x, pending)
        y = self.feed_forward.forward(ctx, h)
        return ops.PendingBranch(y, *self.write_weights[1])


register_part("norm", "streams_rmsnorm", StreamsRMSNorm)
register_part("block", "hyper_connections", HyperConnectionBlock)
