"""A plain, slow restatement of the Zozenex architecture in float64/float32 PyTorch on the CPU: one function per
mechanism, every request by itself, every position from the whole prefix.  It shares no code with the engine; the
tests compare the engine with it.

Notation: ``h`` a token's normed input row, ``t`` / ``i`` / ``j`` positions counted from 0 in a request.
"""

from __future__ import annotations

import math

import torch

DT = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * weight


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def gelu(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, sign: float = 1.0) -> torch.Tensor:
    """``x`` [tokens, heads, channels]: channel ``m`` of the first ``dims`` is paired with ``m + dims/2`` and the pair
    turns by ``sign * position * base ** (-2m / dims)``; channels past ``dims`` pass."""
    if dims == 0:
        return x
    half = dims // 2
    m = torch.arange(half, dtype=DT)
    angle = sign * positions.to(DT)[:, None] * base ** (-2.0 * m / dims)[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def linear_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor) -> torch.Tensor:
    """``S_t = diag(decay_t) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t`` per head from a zero state.
    q, k, decay [tokens, heads, dk]; v [tokens, heads, dv]."""
    tokens, heads, dk = q.shape
    dv = v.shape[-1]
    state = torch.zeros(heads, dk, dv, dtype=DT)
    out = torch.zeros(tokens, heads, dv, dtype=DT)
    for t in range(tokens):
        state = decay[t][:, :, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", state, q[t])
    return out


def retention(h: torch.Tensor, w: dict, cfg: dict, eps: float) -> torch.Tensor:
    heads, dk, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    tokens = h.shape[0]
    q = (h @ w["q"].T).reshape(tokens, heads, dk)
    k = (h @ w["k"].T).reshape(tokens, heads, dk) * dk ** -0.5
    v = (h @ w["v"].T).reshape(tokens, heads, dv)
    decay = torch.tensor(cfg["decay"], dtype=DT)[None, :, None].expand(tokens, heads, dk)
    o = rms(linear_recurrence(q, k, v, decay), eps).reshape(tokens, heads * dv)
    return (o * silu(h @ w["g"].T)) @ w["o"].T


def gated_linear(h: torch.Tensor, w: dict, cfg: dict, eps: float) -> torch.Tensor:
    heads, dk, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    tokens = h.shape[0]
    q = (h @ w["q"].T).reshape(tokens, heads, dk) * dk ** -0.5
    k = (h @ w["k"].T).reshape(tokens, heads, dk)
    v = (h @ w["v"].T).reshape(tokens, heads, dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    decay = torch.sigmoid(z).pow(1.0 / cfg["tau"]).reshape(tokens, heads, dk)
    o = rms_norm(linear_recurrence(q, k, v, decay), w["norm"], eps).reshape(tokens, heads * dv)
    return (o * silu(h @ w["g"].T)) @ w["o"].T


def pooled_sigmoid_attention(h: torch.Tensor, w: dict, cfg: dict) -> torch.Tensor:
    """Sigmoid-weighted attention under a window, with one mean key and mean value for every block of ``pool`` tokens
    that lies wholly before the window; values rotated by their position and the sum turned back by the query's."""
    heads, groups, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    window, pool = cfg["mask"]["size"], cfg["mask"]["pool"]
    rot_dims, base = cfg["rot"]["dims"], cfg["rot"]["base"]
    tokens = h.shape[0]
    positions = torch.arange(tokens)
    q = rotate_halves((h @ w["q"].T).reshape(tokens, heads, dk), positions, rot_dims, base)
    k = rotate_halves((h @ w["k"].T).reshape(tokens, groups, dk), positions, rot_dims, base)
    v = rotate_halves((h @ w["v"].T).reshape(tokens, groups, dv), positions, dv, base)
    out = torch.zeros(tokens, heads, dv, dtype=DT)
    cap = cfg.get("softcap") or 0.0
    for i in range(tokens):
        first = max(0, i - window + 1)
        blocks = max(0, (i - window + 1) // pool)   # block b is seen if (b + 1) * pool - 1 <= i - window
        keys = [k[first : i + 1]]
        values = [v[first : i + 1]]
        if blocks:
            keys.insert(0, k[: blocks * pool].reshape(blocks, pool, groups, dk).mean(dim=1))
            values.insert(0, v[: blocks * pool].reshape(blocks, pool, groups, dv).mean(dim=1))
        keys_i, values_i = torch.cat(keys), torch.cat(values)
        for head in range(heads):
            g = head // (heads // groups)
            score = (keys_i[:, g] @ q[i, head]) * cfg["scale"]
            if cap:   # no cap where the configuration gives none (or zero)
                score = cap * torch.tanh(score / cap)
            weight = torch.sigmoid(score + w["pb"][head])
            out[i, head] = weight @ values_i[:, g]
    out = rotate_halves(out, positions, dv, base, sign=-1.0)
    return out.reshape(tokens, heads * dv) @ w["o"].T


def parallel_mixer(h: torch.Tensor, w: dict, cfg: dict, eps: float) -> torch.Tensor:
    left = pooled_sigmoid_attention(h, {name[len("left."):]: t for name, t in w.items() if name.startswith("left.")}, cfg["left"])
    right = gated_linear(h, {name[len("right."):]: t for name, t in w.items() if name.startswith("right.")}, cfg["right"], eps)
    return 0.5 * (rms_norm(left, w["left.out"], eps) + rms_norm(right, w["right.out"], eps))


def routed_experts(h: torch.Tensor, w: dict, cfg: dict, choice: torch.Tensor | None = None, slack: list | None = None) -> torch.Tensor:
    """``choice`` ([tokens, top], optional): the experts to use instead of the ones this function would choose (for a comparison with
    an implementation whose rounding may turn a close call); ``slack`` then receives, per token, by how much the best expert left
    out beats the worst one taken in this function's own choice scores (not positive where the choice is the right one)."""
    experts, top, scale = cfg["router"]["experts"], cfg["router"]["top"], cfg["router"]["scale"]
    scores = torch.sigmoid(h @ w["router"].T)
    ranking = scores + w["correction"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(experts), key=lambda e: (-float(ranking[t, e]), e))[:top]
        if choice is not None:
            order = [int(e) for e in choice[t]]
            others = [float(ranking[t, e]) for e in range(experts) if e not in order]
            if slack is not None and others:
                slack.append(max(others) - min(float(ranking[t, e]) for e in order))
        for e in order:
            out[t] += scores[t, e] * scale * (gelu(h[t] @ w[f"e{e}.up"].T) @ w[f"e{e}.down"].T)
    if cfg.get("shared") is not None:
        shared = gelu(h @ w["shared.up"].T) @ w["shared.down"].T
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * shared
    return out


def sub(weights: dict, prefix: str) -> dict:
    return {name[len(prefix):]: tensor for name, tensor in weights.items() if name.startswith(prefix)}


def forward(config: dict, weights: dict, tokens: list[int], layers_out: list | None = None, choices: dict | None = None,
            slack: list | None = None) -> torch.Tensor:
    """Logits ``[tokens, vocab]`` of one request read whole; ``weights`` by checkpoint name, in float64.
    ``layers_out`` (a list) receives the stream after every layer.  ``choices`` (layer -> [tokens, top]) and ``slack``: see
    :func:`routed_experts`."""
    eps = config["norm"]["eps"]
    ids = torch.tensor(tokens, dtype=torch.long)
    x = weights["embed"][ids] + weights["pos"][: len(tokens)]
    for index, layer in enumerate(config["layers"]):
        w = sub(weights, f"l{index}.")
        h = rms_norm(x, w["norm1"], eps)
        mix = sub(w, "mix.")
        if layer["type"] == "retention":
            x = x + retention(h, mix, layer["mixer"], eps)
        elif layer["type"] == "parallel":
            x = x + parallel_mixer(h, mix, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + routed_experts(rms_norm(x, w["norm2"], eps), sub(w, "mlp."), layer["mlp"], None if choices is None else choices[index], slack)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, weights["final.norm"], eps) @ weights["head"].T
