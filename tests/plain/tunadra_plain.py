"""A plain, slow Tunadra forward pass in NumPy: one function per mechanism, float64 throughout.

It imports nothing from the engine and the engine imports nothing from here. ``config`` is the
model's config.json as a dict, ``weights`` maps tensor names to arrays. Every function that
carries something from token to token takes and returns that state explicitly, so a sequence can
be fed whole, in portions or token by token.

Notation: ``T`` tokens, ``D`` the model's width, ``n`` streams; a linear weight is ``[out, in]``
and is applied as ``x @ W.T``.
"""

from __future__ import annotations

import numpy as np

F64 = np.float64


def linear(x: np.ndarray, weight: np.ndarray) -> np.ndarray:
    return x.astype(F64) @ weight.astype(F64).T


def sigmoid(x: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-x))


def silu(x: np.ndarray) -> np.ndarray:
    return x * sigmoid(x)


def unit_rms(x: np.ndarray, eps: float) -> np.ndarray:
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    return unit_rms(x.astype(F64), eps) * weight.astype(F64)


# -- embedding ----------------------------------------------------------------------------------------


def sinusoid(positions, width: int) -> np.ndarray:
    """``[T, width]``: column 2i is ``sin(p f_i)``, column 2i + 1 is ``cos(p f_i)``, ``f_i = 10000^(-2i / width)``."""
    p = np.asarray(positions, dtype=F64)[:, None]
    i = np.arange(width // 2, dtype=F64)[None, :]
    angle = p * 10000.0 ** (-2.0 * i / width)
    out = np.zeros((p.shape[0], width), dtype=F64)
    out[:, 0::2] = np.sin(angle)
    out[:, 1::2] = np.cos(angle)
    return out


def embed(table: np.ndarray, tokens, positions, scale: float) -> np.ndarray:
    rows = table[np.asarray(tokens, dtype=np.int64)].astype(F64) * scale
    return rows + sinusoid(positions, table.shape[1])


# -- streams ------------------------------------------------------------------------------------------


def streams_read(xs: np.ndarray, w_in: np.ndarray) -> np.ndarray:
    """``xs`` is ``[n, T, D]``; what a sublayer reads is ``sum_s w_in[s] xs[s]``."""
    return np.einsum("s,std->td", w_in.astype(F64), xs)


def streams_write(xs: np.ndarray, y: np.ndarray, w_mix: np.ndarray, w_out: np.ndarray) -> np.ndarray:
    """All streams at once from the old ones: ``new[t] = sum_s w_mix[s, t] xs[s] + w_out[t] y``."""
    return np.einsum("sr,std->rtd", w_mix.astype(F64), xs) + w_out.astype(F64)[:, None, None] * y[None]


# -- the recurrent mixer ------------------------------------------------------------------------------


def wkv_mixer(h: np.ndarray, w: dict, prefix: str, heads: int, dim: int, eps: float, state=None):
    """Time mixing with a matrix state per head. ``state`` is ``(previous token's h [D], S [heads, dim, dim])``
    or None at a sequence's start. Returns ``(output [T, D], state)``."""
    h = h.astype(F64)
    t_count, width = h.shape

    def get(name):
        return w[prefix + name].astype(F64)

    previous, s = (np.zeros(width, F64), np.zeros((heads, dim, dim), F64)) if state is None else (state[0].copy(), state[1].copy())
    bonus = get("u").reshape(heads, dim)
    out = np.zeros((t_count, heads * dim), F64)
    for t in range(t_count):
        x = h[t]
        shifted = {name: x + (previous - x) * get("mu." + name) for name in "rkvgw"}
        r = (get("r") @ shifted["r"]).reshape(heads, dim)
        k = (get("k") @ shifted["k"]).reshape(heads, dim)
        v = (get("v") @ shifted["v"]).reshape(heads, dim)
        gate = silu(get("g") @ shifted["g"])
        decay = np.exp(-np.exp(get("w2") @ np.tanh(get("w1") @ shifted["w"]) + get("w0"))).reshape(heads, dim)
        o = np.zeros((heads, dim), F64)
        for n in range(heads):
            kv = np.outer(k[n], v[n])
            o[n] = (s[n] + bonus[n][:, None] * kv).T @ r[n]
            s[n] = decay[n][:, None] * s[n] + kv
        o = unit_rms(o, eps).reshape(-1)
        out[t] = o * get("norm") * gate
        previous = x
    return out @ get("o").T, (previous, s)


# -- attention ----------------------------------------------------------------------------------------


def attention_project(h: np.ndarray, w: dict, prefix: str, heads: int, kv_heads: int, dim: int, vdim: int, eps: float):
    """Queries and keys as unit-RMS vectors per head, raw values, and the per-head gate."""
    h = h.astype(F64)
    t = h.shape[0]
    q = unit_rms((h @ w[prefix + "q"].astype(F64).T).reshape(t, heads, dim), eps)
    k = unit_rms((h @ w[prefix + "k"].astype(F64).T).reshape(t, kv_heads, dim), eps)
    v = (h @ w[prefix + "v"].astype(F64).T).reshape(t, kv_heads, vdim)
    gate = sigmoid(h @ w[prefix + "g"].astype(F64).T)
    return q, k, v, gate


def causal_attention(q: np.ndarray, keys: np.ndarray, values: np.ndarray, first_position: int, scale: float) -> np.ndarray:
    """``q [T, H, dim]`` at positions ``first_position ..`` over ``keys [P, G, dim]``, ``values [P, G, vdim]`` that
    hold every position up to the last query's; query head n uses key/value head ``n // (H / G)``."""
    t, heads, _ = q.shape
    share = heads // keys.shape[1]
    out = np.zeros((t, heads, values.shape[-1]), F64)
    for n in range(heads):
        g = n // share
        for i in range(t):
            seen = first_position + i + 1
            scores = keys[:seen, g] @ q[i, n] * scale
            e = np.exp(scores - scores.max())
            out[i, n] = (e / e.sum()) @ values[:seen, g]
    return out


def attention_mixer(h, w, prefix, sizes, eps, first_position=0, cache=None, v_first=None, mixes=False):
    """``cache`` is ``(keys, values)`` of the earlier positions or None. With ``mixes`` the values become
    ``(1 - l) v + l v_first`` before they are cached (``v_first [T, G, vdim]``: the first such layer's
    values of the same tokens). Returns ``(output, cache, this layer's raw values)``."""
    heads, kv_heads, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    q, k, v, gate = attention_project(h, w, prefix, heads, kv_heads, dim, vdim, eps)
    raw = v
    if mixes:
        lam = float(np.asarray(w[prefix + "vmix"], dtype=F64))
        v = (1.0 - lam) * v + lam * v_first
    keys = k if cache is None else np.concatenate([cache[0], k])
    values = v if cache is None else np.concatenate([cache[1], v])
    o = causal_attention(q, keys, values, first_position, float(sizes["scale"])) * gate[:, :, None]
    return o.reshape(h.shape[0], heads * vdim) @ w[prefix + "o"].astype(F64).T, (keys, values), raw


# -- feed-forward ---------------------------------------------------------------------------------------


def clamped_expert(h: np.ndarray, w: dict, prefix: str, limit: float) -> np.ndarray:
    g = np.minimum(linear(h, w[prefix + "gate"]), limit)
    u = np.clip(linear(h, w[prefix + "up"]), -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[prefix + "down"].astype(F64).T


def route(scores: np.ndarray, top: int, group_count: int, group_keep: int) -> np.ndarray:
    """Indices of the ``top`` largest scores among the experts of the ``group_keep`` best of ``group_count``
    equal groups of neighbours; a group's score is the sum of its two largest."""
    experts = scores.shape[0]
    size = experts // group_count
    grouped = scores.reshape(group_count, size)
    group_score = np.sort(grouped, axis=1)[:, -2:].sum(axis=1)
    kept = np.argsort(-group_score, kind="stable")[:group_keep]
    allowed = np.zeros(experts, dtype=bool)
    for g in kept:
        allowed[g * size : (g + 1) * size] = True
    masked = np.where(allowed, scores, -np.inf)
    return np.argsort(-masked, kind="stable")[:top]


def route_margin(scores: np.ndarray, top: int, group_count: int, group_keep: int) -> float:
    """How far the choice is from another one: the smaller of the gap between the last kept and the first
    dropped group's score and the gap between the last chosen and the first unchosen allowed score."""
    experts = scores.shape[0]
    size = experts // group_count
    group_score = np.sort(np.sort(scores.reshape(group_count, size), axis=1)[:, -2:].sum(axis=1))[::-1]
    margin = group_score[group_keep - 1] - group_score[group_keep] if group_keep < group_count else np.inf
    chosen = set(route(scores, experts, group_count, group_keep)[: group_keep * size].tolist())
    allowed = np.sort(scores[sorted(chosen)])[::-1]
    if top < len(allowed):
        margin = min(margin, allowed[top - 1] - allowed[top])
    return float(margin)


def moe(h: np.ndarray, w: dict, prefix: str, mlp: dict, margins: list | None = None, choices=None, free: list | None = None) -> np.ndarray:
    """``margins`` receives, per token, how close the router's choice was (see :func:`route_margin`) and
    ``free`` the choice itself; with ``choices`` (``[T, top]``) the experts are those instead, weighted by
    their own scores as if they had been chosen."""
    h = h.astype(F64)
    router = mlp["router"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    scores = sigmoid(linear(h, w[prefix + "router"]))
    if margins is not None:
        margins.append(np.array([route_margin(row, router["top"], groups["count"], groups["keep"]) for row in scores]))
    if free is not None:
        free.append(np.array([route(row, router["top"], groups["count"], groups["keep"]) for row in scores]))
    out = np.zeros((h.shape[0], w[prefix + "e0.down"].shape[0]), F64)
    for t in range(h.shape[0]):
        chosen = route(scores[t], router["top"], groups["count"], groups["keep"]) if choices is None else np.asarray(choices[t], dtype=np.int64)
        weights = scores[t, chosen] / (scores[t, chosen].sum() + 1e-20) * router["scale"]
        for e, weight in zip(chosen, weights):
            out[t] += weight * clamped_expert(h[t : t + 1], w, f"{prefix}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out += clamped_expert(h, w, prefix + "shared.", mlp["shared"]["limit"])
    return out


# -- the model ------------------------------------------------------------------------------------------


def softcap(logits: np.ndarray, cap: float) -> np.ndarray:
    return cap * np.tanh(logits / cap)


class Sequence:
    """What one sequence carries between calls of :func:`forward`."""

    def __init__(self) -> None:
        self.length = 0
        self.layers: dict[int, object] = {}


def forward(config: dict, w: dict, tokens, seq: Sequence | None = None, layer_sums: list | None = None, margins: list | None = None,
            choices: dict | None = None, free: list | None = None) -> np.ndarray:
    """Feeds ``tokens`` as the next tokens of ``seq`` (a fresh sequence if None); returns logits ``[T, vocab]``.
    ``layer_sums`` receives the sum of the streams after every layer, ``margins`` and ``free`` one array per
    routed layer with every token's distance from another choice of experts and the choice; ``choices``
    (layer index -> ``[T, top]``) replaces the routers' choices."""
    seq = Sequence() if seq is None else seq
    eps = config["norm"]["eps"]
    n = int(config.get("streams", 1))
    positions = np.arange(seq.length, seq.length + len(tokens))
    x0 = embed(w["embed"], tokens, positions, config["embedding"]["scale"])
    xs = np.stack([x0] * n)
    v_first = None

    def sublayer(xs, prefix, q, fn):
        if "streams" in config:
            w_in, w_mix, w_out = (w[f"{prefix}hc{q}.{name}"] for name in ("in", "mix", "out"))
        else:
            w_in, w_mix, w_out = np.ones(1), np.ones((1, 1)), np.ones(1)
        y = fn(rms_norm(streams_read(xs, w_in), w[f"{prefix}norm{q}"], eps))
        return streams_write(xs, y, w_mix, w_out)

    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        sizes = layer["mixer"]

        def mixer(h):
            nonlocal v_first
            if layer["type"] == "wkv":
                y, seq.layers[index] = wkv_mixer(h, w, prefix + "mix.", sizes["heads"], sizes["dim"], eps, seq.layers.get(index))
                return y
            mixes = bool(sizes.get("v_mix")) and v_first is not None
            y, seq.layers[index], raw = attention_mixer(
                h, w, prefix + "mix.", sizes, eps, seq.length, seq.layers.get(index), v_first, mixes
            )
            if sizes.get("v_mix") and v_first is None:
                v_first = raw
            return y

        xs = sublayer(xs, prefix, 1, mixer)
        if layer.get("mlp") is not None:
            xs = sublayer(xs, prefix, 2, lambda h: moe(h, w, prefix + "mlp.", layer["mlp"], margins, None if choices is None else choices[index], free))
        if layer_sums is not None:
            layer_sums.append(xs.sum(axis=0))
    seq.length += len(tokens)
    h = rms_norm(xs.sum(axis=0), w["final.norm"], eps)
    return softcap(linear(h, w["head"]), config["logit_softcap"])


def greedy(config: dict, w: dict, prompt, count: int) -> list[int]:
    """``count`` tokens by arg-max, each from a forward pass over everything so far."""
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(np.argmax(forward(config, w, tokens)[-1])))
    return tokens[len(prompt):]
