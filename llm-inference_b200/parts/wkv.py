"""A recurrent mixer: a matrix state per head with a decay per key channel and a bonus for the current token."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import Part, StateSpec, register_part
from .context import CacheView, StepContext

BLENDS = ("r", "k", "v", "g", "w")


class WKVMixer(Part):
    """With ``h'`` the previous token's input (zeros for a request's first token), each of five
    projections reads its own blend ``h + (h' - h) * mu_s``: ``r, k, v`` (``heads x dim`` each),
    ``gate = silu(W_g .)`` and the decay ``w = exp(-exp(W_w2 tanh(W_w1 .) + w0))`` per head and key
    channel. Per head a state ``S [dim, dim]`` (32-bit, zero at a request's start) is carried from
    token to token: ``o = (S + diag(u) k v^T)^T r`` (the bonus ``u`` applies to the current token only),
    then ``S = diag(w) S + k v^T``. Each head's ``o`` is divided by its root mean square, times ``norm``
    (per channel), times the gate; then ``W_o``.

    Per-request state: ``S`` and the last input ``h``. The four equal-shaped projections are one
    batched product over their blends; the decay's low-rank pair is two small products, the second
    with a 32-bit result; decays, the bonus and the recurrence are 32-bit. The inner size of the
    low-rank pair is the checkpoint's (``decay_rank`` only serves to draw random weights). Tensor
    names are ``prefix + mu.{r,k,v,g,w} | r | k | v | g | w1 | w2 | w0 | u | norm | o``."""

    def __init__(self, *, prefix: str, hidden_size: int, heads: int, dim: int, eps: float, decay_rank: int | None = None) -> None:
        self.prefix, self.hidden_size, self.heads, self.dim, self.eps = prefix, hidden_size, int(heads), int(dim), float(eps)
        self.decay_rank = -1 if decay_rank is None else int(decay_rank)
        self.dtype = torch.bfloat16
        self.mu = self.w_rkvg = self.w_low = self.w_high = self.w_o = self.w0 = self.bonus = self.norm_weight = None

    def cache_spec(self) -> StateSpec:
        return StateSpec(((self.heads, self.dim, self.dim), (self.hidden_size,)), (torch.float32, self.dtype))

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, inner = self.prefix, self.hidden_size, self.heads * self.dim
        specs = [TensorSpec(p + "mu." + s, (d,), init="half_plus_normal") for s in BLENDS]
        specs += [TensorSpec(p + s, (inner, d)) for s in ("r", "k", "v", "g")]
        specs += [
            TensorSpec(p + "w1", (self.decay_rank, d)), TensorSpec(p + "w2", (inner, self.decay_rank)), TensorSpec(p + "w0", (inner,)),
            TensorSpec(p + "u", (self.heads, self.dim)), TensorSpec(p + "norm", (inner,), init="one_plus_normal"),
            TensorSpec(p + "o", (d, inner)),
        ]
        return specs

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix
        self.dtype = dtype

        def get(name: str, to=dtype) -> torch.Tensor:
            return tensors[p + name].to(device=device, dtype=to).contiguous()

        f32 = torch.float32
        self.mu = torch.stack([get("mu." + s, f32) for s in BLENDS]).contiguous()
        self.w_rkvg = torch.stack([get(s) for s in ("r", "k", "v", "g")]).contiguous()
        self.w_low, self.w_high, self.w_o = get("w1"), get("w2"), get("o")
        self.w0, self.bonus, self.norm_weight = get("w0", f32), get("u", f32).reshape(-1).contiguous(), get("norm", f32)

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_rkvg, self.w_low, self.w_high, self.w_o))

    def forward(self, ctx: StepContext, cache: CacheView, h: torch.Tensor) -> torch.Tensor:
        t, heads, dim = ctx.num_tokens, self.heads, self.dim
        inner = heads * dim
        state, shift = cache.state
        f32 = torch.float32
        blends = ops.wkv_shift_mix(ctx, h, shift, self.mu, ctx.buffer("wkv_blends", (len(BLENDS), t, self.hidden_size)))
        proj = ops.linear_per_head(ctx, blends[:4], self.w_rkvg, ctx.buffer("wkv_proj", (4, t, inner)))
        low = ops.linear(ctx, blends[4], self.w_low, ctx.buffer("wkv_low", (t, self.w_low.shape[0])))
        low = ops.tanh_rows(ctx, low)
        log_decay = ops.linear(ctx, low, self.w_high, ctx.buffer("wkv_log_decay", (t, inner), f32))
        r, k, v = (ctx.buffer("wkv_" + name, (t, inner), f32) for name in ("r32", "k32", "v32"))
        decay, bonus = ctx.buffer("wkv_decay", (t, inner), f32), ctx.buffer("wkv_bonus", (t, heads), f32)
        ops.wkv_prepare(ctx, proj[0], proj[1], proj[2], log_decay, self.w0, self.bonus, heads, dim, r, k, v, decay, bonus)
        o = ops.wkv_recurrence(ctx, r, k, v, bonus, decay, state, ctx.buffer("wkv_o", (t, inner), f32), heads, dim, dim)
        y = ops.wkv_output(ctx, o, self.norm_weight, proj[3], heads, dim, self.eps, ctx.buffer("attn", (t, inner)))
        return ops.linear(ctx, y, self.w_o, ctx.buffer("branch", (t, self.hidden_size)))


register_part("mixer", "wkv", WKVMixer)
