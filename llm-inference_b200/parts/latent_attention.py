"""Attention whose keys and values are expanded from one cached low-rank latent per token."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import KVCacheSpec, Part, PartSpec, build_part, register_part
from .context import CacheView, StepContext


class LatentAttention(Part):
    """Causal attention over cached latents.

    Per token ``W_dkv h`` gives ``rank`` numbers, RMS-normed into the latent ``c``, plus
    ``rot_dim`` numbers that, rotated at the token's position, are a key part shared by all heads;
    only these ``rank + rot_dim`` numbers are cached. Head ``n`` has the query
    ``[q_plain (dim) | q_rot (rot_dim)]`` from ``W_q h``, the key ``[W_uk[n] c | k_rot]`` and the
    value ``W_uv[n] c``; the score is ``(q_plain . W_uk[n] c + q_rot . k_rot) * scale``. Since
    ``q_plain . W_uk[n] c = (W_uk[n]^T q_plain) . c``, the query is carried into the latent space by
    one small product per head, the attention kernel works on the cached rows as they are, and its
    result ``sum_j p_j c_j`` is expanded by ``W_uv[n]`` afterwards. With ``sink`` the softmax's
    denominator also holds ``exp(sink[n])`` (no key, no value, not scaled); with ``gate`` a head's
    output is multiplied by ``sigmoid(W_g h)[n]``. Then ``W_o`` on the concatenated heads.

    The query, latent and gate projections are one matrix product. Tensor names are
    ``prefix + q | dkv | dkv.norm | uk | uv | sink | g | o``."""

    def __init__(self, *, prefix: str, hidden_size: int, heads: int, dim: int, rot_dim: int, vdim: int, rank: int,
                 scale: float, eps: float, position: PartSpec, sink: bool = True, gate: bool = True, window: int = 0) -> None:
        self.prefix, self.hidden_size = prefix, hidden_size
        self.heads, self.dim, self.rot_dim, self.vdim, self.rank = heads, dim, rot_dim, vdim, rank
        self.scale, self.eps, self.window = float(scale), float(eps), int(window)
        self.has_sink, self.has_gate = bool(sink), bool(gate)
        self.position = build_part("position", position)
        self.graph_safe = self.position.graph_safe
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.sink = self.norm_weight = None

    def cache_spec(self) -> KVCacheSpec:
        return KVCacheSpec(1, self.rank + self.rot_dim, self.window, planes=1)

    def tensor_specs(self) -> list[TensorSpec]:
        p, d = self.prefix, self.hidden_size
        specs = [
            TensorSpec(p + "q", (self.heads * (self.dim + self.rot_dim), d)),
            TensorSpec(p + "dkv", (self.rank + self.rot_dim, d)),
            TensorSpec(p + "dkv.norm", (self.rank,), init="one_plus_normal"),
            TensorSpec(p + "uk", (self.heads * self.dim, self.rank)),
            TensorSpec(p + "uv", (self.heads * self.vdim, self.rank)),
            TensorSpec(p + "o", (d, self.heads * self.vdim)),
        ]
        if self.has_sink:
            specs.append(TensorSpec(p + "sink", (self.heads,)))
        if self.has_gate:
            specs.append(TensorSpec(p + "g", (self.heads, d)))
        return specs + self.position.tensor_specs()

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix
        names = ["q", "dkv"] + (["g"] if self.has_gate else [])
        self.w_in = torch.cat([tensors[p + n].to(device=device, dtype=dtype) for n in names]).contiguous()
        # [heads, rank, dim]: the product that carries a query into the latent space reads W_uk[n]^T.
        self.w_uk_t = tensors[p + "uk"].to(device=device, dtype=dtype).view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[p + "uv"].to(device=device, dtype=dtype).view(self.heads, self.vdim, self.rank).contiguous()
        self.w_o = tensors[p + "o"].to(device=device, dtype=dtype).contiguous()
        self.norm_weight = tensors[p + "dkv.norm"].to(device=device, dtype=torch.float32).contiguous()
        self.sink = tensors[p + "sink"].to(device=device, dtype=torch.float32).contiguous() if self.has_sink else None
        self.position.load(tensors, dtype, device)

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_uk_t, self.w_uv, self.w_o))

    def forward(self, ctx: StepContext, cache: CacheView, h: torch.Tensor) -> torch.Tensor:
        t, heads, rank, rot = ctx.num_tokens, self.heads, self.rank, self.rot_dim
        q_width = heads * (self.dim + rot)
        width = self.w_in.shape[0]
        proj = ops.linear(ctx, h, self.w_in, ctx.buffer("latent_in", (t, width)))
        q_rot = ctx.buffer("latent_q_rot", (t, heads * rot))
        self.position.apply_latent(ctx, cache, proj, 0, q_width, heads, self.dim, rank, self.norm_weight, self.eps, q_rot)
        q_plain = proj[:, :q_width].view(t, heads, self.dim + rot)[:, :, : self.dim].transpose(0, 1)
        q_lat = ops.linear_per_head(ctx, q_plain, self.w_uk_t, ctx.buffer("latent_q", (heads, t, rank)))
        gate = proj[:, q_width + rank + rot :] if self.has_gate else None
        mixed = ctx.buffer("latent_out", (heads, t, rank))
        self.attend(ctx, cache, q_lat, q_rot, gate, mixed)
        attn = ctx.buffer("attn", (t, heads * self.vdim))
        ops.linear_per_head(ctx, mixed, self.w_uv, attn.view(t, heads, self.vdim).transpose(0, 1))
        return ops.linear(ctx, attn, self.w_o, ctx.buffer("branch", (t, self.hidden_size)))

    def attend(self, ctx: StepContext, cache: CacheView, q_lat, q_rot, gate, out) -> None:
        from . import attention_dispatch

        attention_dispatch.attend_latent(ctx, cache, q_lat, q_rot, self.sink, gate, out, self.heads, self.rank, self.rot_dim, self.scale)


register_part("mixer", "latent_attention", LatentAttention)
