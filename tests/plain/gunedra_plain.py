"""A plain, slow Gunedra forward pass in NumPy: whole sequences, no cache, one function per mechanism.

It imports nothing from the engine and the engine imports nothing from here. Arithmetic is
float64 throughout, so it stands above both the engine's float32 path and its bfloat16 path.
``config`` is the model's config.json as a dict, ``weights`` maps tensor names to arrays.

Notation: ``T`` tokens, ``D`` the model's width, a linear weight is ``[out, in]`` and is applied
as ``x @ W.T``.
"""

from __future__ import annotations

import math

import numpy as np

F64 = np.float64


def linear(x: np.ndarray, weight: np.ndarray) -> np.ndarray:
    return x.astype(F64) @ weight.astype(F64).T


def sigmoid(x: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-x))


def silu(x: np.ndarray) -> np.ndarray:
    return x * sigmoid(x)


def softplus(x: np.ndarray) -> np.ndarray:
    return np.logaddexp(0.0, x)


def rms(x: np.ndarray, eps: float) -> np.ndarray:
    """``sqrt(mean(x^2) + eps)`` over the last axis, the epsilon inside the root."""
    return np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def embed(table: np.ndarray, tokens, scale: float) -> np.ndarray:
    """``table[token] * scale``."""
    return table[np.asarray(tokens, dtype=np.int64)].astype(F64) * scale


def grouped_rms_norm(x: np.ndarray, weight: np.ndarray, groups: int, eps: float) -> np.ndarray:
    """The vector is cut into ``groups`` equal consecutive parts, each divided by its own root
    mean square; the whole is then multiplied by ``weight``."""
    t, d = x.shape
    parts = x.astype(F64).reshape(t, groups, d // groups)
    return (parts / rms(parts, eps)).reshape(t, d) * weight.astype(F64)


def rotate_interleaved(x: np.ndarray, positions, base: float, dims: int) -> np.ndarray:
    """Rotary encoding of ``[T, ..., n]`` over its first ``dims`` dims, dim 2i paired with
    2i + 1: ``(u, v) -> (u cos a - v sin a, v cos a + u sin a)``, ``a = p * base^(-2i/dims)``."""
    x = x.astype(F64).copy()
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half, dtype=F64) / dims)
    angle = np.asarray(positions, dtype=F64)[:, None] * freq[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    cos, sin = np.cos(angle).reshape(shape), np.sin(angle).reshape(shape)
    u, v = x[..., 0:dims:2].copy(), x[..., 1:dims:2].copy()
    x[..., 0:dims:2] = u * cos - v * sin
    x[..., 1:dims:2] = v * cos + u * sin
    return x


def sink_softmax_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, sink: np.ndarray, scale: float) -> np.ndarray:
    """Causal attention of ``q [T, H, dk]`` over ``k [T, H, dk]``, ``v [T, H, dv]``. The softmax's
    denominator also holds ``exp(sink[h])``: a term with no key and no value, not scaled."""
    t, heads, _ = q.shape
    out = np.zeros((t, heads, v.shape[-1]), dtype=F64)
    for h in range(heads):
        scores = (q[:, h] @ k[:, h].T) * scale
        for i in range(t):
            row = scores[i, : i + 1]
            top = max(row.max(), float(sink[h]))
            e = np.exp(row - top)
            out[i, h] = (e @ v[: i + 1, h]) / (e.sum() + math.exp(float(sink[h]) - top))
    return out


def latent_attention(config: dict, weights: dict, prefix: str, mixer: dict, h: np.ndarray, positions) -> np.ndarray:
    """Attention whose keys and values are expanded from one low-rank latent per token plus one
    rotated key part that all heads share; sink in the softmax; a sigmoid gate per head."""
    t = h.shape[0]
    heads, dim, rot_dim, vdim, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    eps = config["norm"]["eps"]
    base, dims = mixer["rot"]["base"], mixer["rot"]["dims"]
    q = linear(h, weights[prefix + "q"]).reshape(t, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate_interleaved(q[..., dim:], positions, base, dims)
    down = linear(h, weights[prefix + "dkv"])
    latent = down[:, :rank]
    latent = latent / rms(latent, eps) * weights[prefix + "dkv.norm"].astype(F64)
    k_rot = rotate_interleaved(down[:, rank:], positions, base, dims)
    k_plain = linear(latent, weights[prefix + "uk"]).reshape(t, heads, dim)
    values = linear(latent, weights[prefix + "uv"]).reshape(t, heads, vdim)
    keys = np.concatenate([k_plain, np.broadcast_to(k_rot[:, None, :], (t, heads, rot_dim))], axis=-1)
    queries = np.concatenate([q_plain, q_rot], axis=-1)
    out = sink_softmax_attention(queries, keys, values, weights[prefix + "sink"].astype(F64), mixer["scale"])
    gate = sigmoid(linear(h, weights[prefix + "g"]))  # [T, H]
    out = out * gate[:, :, None]
    return linear(out.reshape(t, heads * vdim), weights[prefix + "o"])


def short_convolution(x: np.ndarray, taps: np.ndarray) -> np.ndarray:
    """Causal convolution over time per channel: ``y[t, c] = sum_j taps[c, j] x[t - (n-1) + j, c]``
    (the last column weighs the current token), zeros before the start, then silu."""
    t, _ = x.shape
    n = taps.shape[1]
    padded = np.concatenate([np.zeros((n - 1, x.shape[1]), dtype=F64), x.astype(F64)], axis=0)
    y = np.zeros_like(x, dtype=F64)
    for j in range(n):
        y += padded[j : j + t] * taps[:, j].astype(F64)[None, :]
    return silu(y)


def unit(x: np.ndarray) -> np.ndarray:
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)


def gated_delta_rule(q, k, v, beta, decay) -> np.ndarray:
    """One head. ``q, k, decay [T, dk]``, ``v [T, dv]``, ``beta [T]``; the state ``S [dk, dv]``
    starts at zero. Per token: ``S = decay[:, None] * S``; ``u = beta (v - S^T k)``;
    ``S = S + k u^T``; ``o = S^T q``."""
    t, dk = k.shape
    state = np.zeros((dk, v.shape[1]), dtype=F64)
    out = np.zeros((t, v.shape[1]), dtype=F64)
    for i in range(t):
        state = decay[i][:, None] * state
        u = beta[i] * (v[i] - state.T @ k[i])
        state = state + np.outer(k[i], u)
        out[i] = state.T @ q[i]
    return out


def channel_delta(config: dict, weights: dict, prefix: str, mixer: dict, h: np.ndarray) -> np.ndarray:
    """The gated delta rule with one decay per head and key channel."""
    t = h.shape[0]
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    eps = config["norm"]["eps"]
    q = short_convolution(linear(h, weights[prefix + "q"]), weights[prefix + "q.conv"]).reshape(t, kv_heads, dim)
    k = short_convolution(linear(h, weights[prefix + "k"]), weights[prefix + "k.conv"]).reshape(t, kv_heads, dim)
    v = short_convolution(linear(h, weights[prefix + "v"]), weights[prefix + "v.conv"]).reshape(t, heads, vdim)
    q = unit(q) * dim**-0.5
    k = unit(k)
    beta = sigmoid(linear(h, weights[prefix + "b"]))  # [T, heads]
    step = softplus(linear(linear(h, weights[prefix + "a1"]), weights[prefix + "a2"]) + weights[prefix + "dt_bias"].astype(F64))
    rate = np.exp(weights[prefix + "A_log"].astype(F64))  # [heads]
    decay = np.exp(-rate[None, :, None] * step.reshape(t, heads, dim))
    gate = sigmoid(linear(linear(h, weights[prefix + "g1"]), weights[prefix + "g2"])).reshape(t, heads, vdim)
    share = heads // kv_heads
    out = np.zeros((t, heads, vdim), dtype=F64)
    for head in range(heads):
        o = gated_delta_rule(q[:, head // share], k[:, head // share], v[:, head], beta[:, head], decay[:, head])
        out[:, head] = o / rms(o, eps) * weights[prefix + "norm"].astype(F64) * gate[:, head]
    return linear(out.reshape(t, heads * vdim), weights[prefix + "o"])


def poly_norm_feed_forward(config: dict, weights: dict, prefix: str, h: np.ndarray) -> np.ndarray:
    """``down(a N(z) + b N(z^2) + c N(z^3) + e)`` with ``z = up(h)``, powers element by element
    and ``N`` dividing a token's vector by its root mean square."""
    eps = config["norm"]["eps"]
    z = linear(h, weights[prefix + "up"])
    a, b, c, e = (float(x) for x in weights[prefix + "act"].astype(F64))
    z2, z3 = z * z, z * z * z
    act = a * z / rms(z, eps) + b * z2 / rms(z2, eps) + c * z3 / rms(z3, eps) + e
    return linear(act, weights[prefix + "down"])


def forward(config: dict, weights: dict, tokens, return_layers: bool = False):
    """Logits ``[T, vocab]`` of one sequence (positions from 0); with ``return_layers`` also the
    stream that leaves every layer, ``[layers, T, D]``."""
    norm = config["norm"]
    mult = config["residual_mult"]
    positions = np.arange(len(tokens))
    x = embed(weights["embed"], tokens, config["embedding"]["scale"])
    history = [x]
    after = []
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        if layer["type"] == "latent_attention":
            mixed = latent_attention(config, weights, p + "mix.", layer["mixer"], x, positions)
        elif layer["type"] == "channel_delta":
            mixed = channel_delta(config, weights, p + "mix.", layer["mixer"], x)
        else:
            raise ValueError(layer["type"])
        x = x + mult * weights[p + "ls1"].astype(F64) * grouped_rms_norm(mixed, weights[p + "norm1"], norm["groups"], norm["eps"])
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            ff = poly_norm_feed_forward(config, weights, p + "mlp.", x)
            x = x + mult * weights[p + "ls2"].astype(F64) * grouped_rms_norm(ff, weights[p + "norm2"], norm["groups"], norm["eps"])
        history.append(x)
        mix = weights[p + "dwa"].astype(F64)
        x = sum(mix[j] * history[j] for j in range(index + 2))
        after.append(x)
    x = grouped_rms_norm(x, weights["final.norm"], norm["groups"], norm["eps"])
    logits = linear(x, weights["embed"])
    return (logits, np.stack(after)) if return_layers else logits


def greedy(config: dict, weights: dict, prompt, count: int) -> list[int]:
    tokens = list(prompt)
    out = []
    for _ in range(count):
        token = int(np.argmax(forward(config, weights, tokens)[-1]))
        out.append(token)
        tokens.append(token)
    return out
