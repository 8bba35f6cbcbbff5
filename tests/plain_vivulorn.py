"""A plain, slow restatement of the Vivulorn design in NumPy float64: one function per mechanism,
whole sequences at once, no cache and no batching.  It shares no code with the package; the tests
compare the engine's logits (prefill, decoding through the cache, portions, mixed batches) with it.

Notation: ``x`` is ``[tokens, width]``; linear weights are ``[out, in]`` and applied as ``x @ W.T``.
Tensor names are the checkpoint's: ``l<i>.mix.q``, ``l<i>.mlp.up.b`` and so on.
"""

from __future__ import annotations

import math

import numpy as np

__all__ = [
    "delta_mixer", "delta_rule", "dense_mlp", "forward", "gated_attention", "gelu_erf", "latent_attention", "layer", "layer_norm",
    "layer_runs", "rms_norm", "rotate_half", "rotate_pairs", "short_convolution", "sink_softmax", "softcap", "yarn_frequencies",
]

UNIT_EPS = 1e-6  # the design fixes the epsilon under the root that makes q and k unit vectors
_erf = np.vectorize(math.erf, otypes=[np.float64])


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_erf(z):
    return 0.5 * z * (1.0 + _erf(z / math.sqrt(2.0)))


def rms_norm(x, weight, eps):
    """``x / sqrt(mean(x^2) + eps) * weight`` over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * weight


def layer_norm(x, weight, bias, eps):
    """``(x - mean) / sqrt(var + eps) * weight + bias`` with the variance as the mean squared deviation."""
    centred = x - x.mean(axis=-1, keepdims=True)
    return centred / np.sqrt(np.mean(centred * centred, axis=-1, keepdims=True) + eps) * weight + bias


def plain_frequencies(dims, base):
    return base ** (-2.0 * np.arange(dims // 2) / dims)


def yarn_frequencies(dims, base, scaling):
    """Frequencies and the factor on cos and sin: each frequency is blended between itself and itself over ``factor``
    by a ramp over the pair index between the pairs that turn ``fast`` and ``slow`` times within ``original`` positions."""
    freq = plain_frequencies(dims, base)
    if scaling is None:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def _cos_sin(positions, freq, magnitude):
    angle = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    return (np.cos(angle) * magnitude)[:, None, :], (np.sin(angle) * magnitude)[:, None, :]


def rotate_half(x, positions, dims, freq, magnitude=1.0):
    """Rotation of the first ``dims`` channels of ``x [tokens, heads, dim]``, channel ``i`` paired with ``i + dims/2``."""
    out = x.copy()
    half = dims // 2
    if half == 0:
        return out
    cos, sin = _cos_sin(positions, freq, magnitude)
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def rotate_pairs(x, positions, dims, freq, magnitude=1.0):
    """Rotation of the first ``dims`` channels of ``x [tokens, heads, dim]``, channel ``2i`` paired with ``2i + 1``."""
    out = x.copy()
    if dims == 0:
        return out
    cos, sin = _cos_sin(positions, freq, magnitude)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def causal_mask(n):
    return np.arange(n)[None, :] <= np.arange(n)[:, None]


def sink_softmax(scores, mask, sink=None):
    """Softmax over the visible keys of ``scores [..., queries, keys]``; with ``sink`` (broadcastable to
    ``[..., queries, 1]``) the denominator holds ``exp(sink)`` as well, once, with no value behind it."""
    scores = np.where(mask, scores, -np.inf)
    top = scores.max(axis=-1, keepdims=True)
    if sink is not None:
        top = np.maximum(top, sink)
    weights = np.exp(scores - top)
    total = weights.sum(axis=-1, keepdims=True)
    if sink is not None:
        total = total + np.exp(sink - top)
    return weights / total


def gated_attention(h, w, prefix, c, eps, positions=None):
    """Grouped softmax attention: RMS norm of the whole q and the whole k projection, rotation in halves with blended
    frequencies, causal softmax, a sigmoid gate from the mixer's input on the concatenated heads, out-projection."""
    n = h.shape[0]
    positions = np.arange(n) if positions is None else positions
    heads, groups, dim, vdim = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = rms_norm(h @ w[prefix + "q"].T, w[prefix + "q.norm"], eps).reshape(n, heads, dim)
    k = rms_norm(h @ w[prefix + "k"].T, w[prefix + "k.norm"], eps).reshape(n, groups, dim)
    v = (h @ w[prefix + "v"].T).reshape(n, groups, vdim)
    rot = c["rot"]
    freq, magnitude = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    q = rotate_half(q, positions, rot["dims"], freq, magnitude)
    k = rotate_half(k, positions, rot["dims"], freq, magnitude)
    per_group = heads // groups
    out = np.zeros((n, heads, vdim))
    mask = causal_mask(n)
    for head in range(heads):
        group = head // per_group
        scores = q[:, head] @ k[:, group].T * c["scale"]
        out[:, head] = sink_softmax(scores, mask) @ v[:, group]
    gate = sigmoid(h @ w[prefix + "g"].T)
    return (out.reshape(n, heads * vdim) * gate) @ w[prefix + "o"].T


def latent_attention(h, w, prefix, c, eps, positions=None):
    """Attention whose keys and values are projections of one normed latent vector per token, plus one rotated key part
    shared by all heads (pairs of neighbouring channels turn together); the softmax's denominator holds a sink per head."""
    n = h.shape[0]
    positions = np.arange(n) if positions is None else positions
    heads, dim, rot_dim, vdim, rank = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    freq = plain_frequencies(rot_dim, c["rot"]["base"])
    q = (h @ w[prefix + "q"].T).reshape(n, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate_pairs(q[..., dim:], positions, rot_dim, freq)
    down = h @ w[prefix + "dkv"].T
    latent = rms_norm(down[:, :rank], w[prefix + "dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, None, rank:], positions, rot_dim, freq)[:, 0]
    k_plain = (latent @ w[prefix + "uk"].T).reshape(n, heads, dim)
    values = (latent @ w[prefix + "uv"].T).reshape(n, heads, vdim)
    out = np.zeros((n, heads, vdim))
    mask = causal_mask(n)
    for head in range(heads):
        scores = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * c["scale"]
        out[:, head] = sink_softmax(scores, mask, sink=w[prefix + "sink"][head]) @ values[:, head]
    return out.reshape(n, heads * vdim) @ w[prefix + "o"].T


def short_convolution(x, taps_weight, before=None):
    """Causal convolution per channel: ``y[t] = sum_j weight[:, taps - 1 - j] * x[t - j]``, zeros (or ``before``, the
    ``taps - 1`` inputs that came earlier) ahead of the start."""
    n, channels = x.shape
    taps = taps_weight.shape[1]
    ahead = np.zeros((taps - 1, channels)) if before is None else before
    padded = np.concatenate([ahead, x], axis=0)
    out = np.zeros_like(x)
    for j in range(taps):
        out += padded[taps - 1 - j : taps - 1 - j + n] * taps_weight[:, taps - 1 - j]
    return out


def delta_rule(q, k, v, beta, g, state=None):
    """One head: ``S <- g_t S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t``.  ``q, k [n, dk]``, ``v [n, dv]``,
    ``beta, g [n]``.  Returns the read-outs and the last state."""
    n, dk = k.shape
    dv = v.shape[1]
    S = np.zeros((dk, dv)) if state is None else state.copy()
    out = np.zeros((n, dv))
    for t in range(n):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out, S


def delta_mixer(h, w, prefix, c, eps):
    """The gated-delta-rule mixer: convolved, silu'd q, k, v; unit q and k; one decay per head; per-head RMS norm of the
    read-out times a silu gate."""
    n = h.shape[0]
    heads, groups, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = silu(short_convolution(h @ w[prefix + "q"].T, w[prefix + "q.conv"])).reshape(n, groups, dk)
    k = silu(short_convolution(h @ w[prefix + "k"].T, w[prefix + "k.conv"])).reshape(n, groups, dk)
    v = silu(short_convolution(h @ w[prefix + "v"].T, w[prefix + "v.conv"])).reshape(n, heads, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + UNIT_EPS) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + UNIT_EPS)
    beta = sigmoid(h @ w[prefix + "b"].T)
    decay = np.exp(-np.exp(w[prefix + "A_log"]) * softplus(h @ w[prefix + "a"].T + w[prefix + "dt_bias"]))
    per_group = heads // groups
    out = np.zeros((n, heads, dv))
    for head in range(heads):
        group = head // per_group
        out[:, head], _ = delta_rule(q[:, group], k[:, group], v[:, head], beta[:, head], decay[:, head])
    out = rms_norm(out, w[prefix + "norm"], eps)
    gate = silu(h @ w[prefix + "g"].T)
    return (out.reshape(n, heads * dv) * gate) @ w[prefix + "o"].T


def dense_mlp(h, w, prefix):
    hidden = gelu_erf(h @ w[prefix + "up"].T + w[prefix + "up.b"])
    return hidden @ w[prefix + "down"].T + w[prefix + "down.b"]


MIXERS = {"attention": gated_attention, "latent_attention": latent_attention, "delta": delta_mixer}


def layer(x, w, index, entry, eps):
    root = f"l{index}."
    h = layer_norm(x, w[root + "norm1"], w[root + "norm1.b"], eps)
    x = x + MIXERS[entry["type"]](h, w, root + "mix.", entry["mixer"], eps)
    if entry.get("mlp") is not None:
        h = layer_norm(x, w[root + "norm2"], w[root + "norm2.b"], eps)
        x = x + dense_mlp(h, w, root + "mlp.")
    return x


def layer_runs(config):
    """``(layer index, first of a pass)`` for every layer run: the stretch ``loop.start .. loop.stop - 1`` runs
    ``loop.times`` times in a row."""
    count = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return [(index, False) for index in range(count)]
    runs = [(index, False) for index in range(loop["start"])]
    for _ in range(loop["times"]):
        runs += [(index, index == loop["start"]) for index in range(loop["start"], loop["stop"])]
    return runs + [(index, False) for index in range(loop["stop"], count)]


def softcap(logits, cap):
    return cap * np.tanh(logits / cap)


def forward(tokens, w, config, collect=None):
    """Logits ``[tokens, vocab]`` of one sequence.  ``collect``: a list that receives the stream after every layer run."""
    w = {name: np.asarray(value, dtype=np.float64) for name, value in w.items()}
    eps = config["norm"]["eps"]
    x0 = w["embed"][np.asarray(tokens)] * config.get("embedding", {}).get("scale", 1.0)
    x = x0
    for index, first_of_pass in layer_runs(config):
        if first_of_pass:
            x = np.concatenate([x, x0], axis=1) @ w["loop.in"].T
        x = layer(x, w, index, config["layers"][index], eps)
        if collect is not None:
            collect.append(x.copy())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    logits = x @ w["embed"].T
    cap = config.get("logit_softcap")
    return softcap(logits, cap) if cap else logits
