"""An attention mixer without position encoding: unit-RMS queries and keys, values blended across layers, a gate per head."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import KVCacheSpec, Part, register_part
from .context import CacheView, StepContext


def padded_head_size(dim: int, vdim: int) -> int:
    """The row width of the cache: keys (``dim``) and values (``vdim``) share one arena shape, and the
    tensor-core attention kernels take heads of 64 or 128; smaller heads are padded with zeros up to
    those, larger ones to a multiple of 16."""
    need = max(dim, vdim)
    if need <= 64:
        return 64
    if need <= 128:
        return 128
    return (need + 15) // 16 * 16


class GatedAttention(Part):
    """Causal grouped-query attention over a paged cache, positions not entering the scores.

    ``q = W_q h`` (``heads x dim``), ``k = W_k h`` (``kv_heads x dim``), ``v = W_v h`` (``kv_heads x vdim``), no
    biases; with ``qk_norm`` each query and key head is divided by its root mean square (no weight);
    ``softmax(q . k * scale)`` over the keys up to the token's own; query head ``n`` uses key/value head
    ``n // (heads / kv_heads)``. ``values``: ``"publish"`` makes this layer's values available to later
    layers of the step (buffer ``shared_values``), ``"blend"`` replaces ``v`` by ``(1 - l) v + l v_shared``
    (``l`` the scalar tensor ``vmix``; what is cached is the blended value), None does neither. With
    ``gate`` head ``n``'s output is multiplied by ``sigmoid(W_g h)_n``. Then ``W_o``.

    The four projections are one matrix ``[q | k | v | g]``. Tensor names: ``prefix + q | k | v | g | vmix | o``
    (``vmix`` is read past in a layer that does not blend)."""

    def __init__(self, *, prefix: str, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, eps: float,
                 qk_norm: bool = True, gate: bool = True, values: str | None = None, has_blend_tensor: bool = False) -> None:
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads cannot share {kv_heads} kv heads")
        if values not in (None, "publish", "blend"):
            raise ValueError(f"values={values!r} must be None, 'publish' or 'blend'")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.eps, self.qk_norm, self.gate, self.values = float(scale), float(eps), bool(qk_norm), bool(gate), values
        self.has_blend_tensor = bool(has_blend_tensor) or values == "blend"
        self.row_dim = padded_head_size(self.dim, self.vdim)
        self.w_in = self.w_o = self.blend = None

    def cache_spec(self) -> KVCacheSpec:
        return KVCacheSpec(self.kv_heads, self.row_dim, 0)

    def tensor_specs(self) -> list[TensorSpec]:
        p, d = self.prefix, self.hidden_size
        specs = [
            TensorSpec(p + "q", (self.heads * self.dim, d)), TensorSpec(p + "k", (self.kv_heads * self.dim, d)),
            TensorSpec(p + "v", (self.kv_heads * self.vdim, d)), TensorSpec(p + "o", (d, self.heads * self.vdim)),
        ]
        if self.gate:
            specs.append(TensorSpec(p + "g", (self.heads, d)))
        if self.has_blend_tensor:
            specs.append(TensorSpec(p + "vmix", (), init="half_plus_normal", optional=self.values != "blend"))
        return specs

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix
        names = ["q", "k", "v"] + (["g"] if self.gate else [])
        self.w_in = torch.cat([tensors[p + n].to(device=device, dtype=dtype) for n in names]).contiguous()
        self.w_o = tensors[p + "o"].to(device=device, dtype=dtype).contiguous()
        if self.values == "blend":
            self.blend = tensors[p + "vmix"].to(device=device, dtype=torch.float32).reshape(1).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_o.element_size()

    def forward(self, ctx: StepContext, cache: CacheView, h: torch.Tensor) -> torch.Tensor:
        t, heads, kvh, row = ctx.num_tokens, self.heads, self.kv_heads, self.row_dim
        proj = ops.linear(ctx, h, self.w_in, ctx.buffer("gated_proj", (t, self.w_in.shape[0])))
        q = ctx.buffer("q", (t, heads * row))
        shared = ctx.buffer("shared_values", (t, kvh * self.vdim)) if self.values else None
        ops.norm_kv_write(
            ctx, cache, proj, q, heads, kvh, self.dim, self.vdim, row, self.qk_norm, self.eps, shared_values=shared,
            blend=self.blend if self.values == "blend" else None, publish=self.values == "publish",
        )
        attn = ctx.buffer("attn_rows", (t, heads * row))
        from . import attention_dispatch

        attention_dispatch.attend(ctx, cache, q, attn, heads, kvh, row, self.scale)
        gate_offset = heads * self.dim + kvh * (self.dim + self.vdim)
        gated = ops.head_gate(ctx, attn, proj if self.gate else None, gate_offset, heads, self.vdim, row, ctx.buffer("attn", (t, heads * self.vdim)))
        return ops.linear(ctx, gated, self.w_o, ctx.buffer("branch", (t, self.hidden_size)))


register_part("mixer", "gated_attention", GatedAttention)
