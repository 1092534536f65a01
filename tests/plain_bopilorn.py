"""Plain, slow Bopilorn decoder: the oracle of the tests of that architecture.

Whole sequences only, no cache, no kernels, one function per mechanism.  It shares no code with the
package: it reads tensors by their checkpoint names out of a ``dict`` and sizes and constants out of
the ``config.json`` dictionary.  ``dtype`` is the arithmetic (float64 by default, so that the oracle's
own rounding never shows).

Notation.  T tokens at positions 0..T-1, stream x [T, W] = E[token] * embedding.scale.  A layer is
x <- x + N1b(mixer(N1(x))), then (if it has a feed-forward) x <- x + N2b(ff(N2(x))), every N a
layer norm with a weight and no bias.  The mixer is grouped-query softmax attention whose values are
unit-normalised and turned by their positions (and whose outputs are turned back); the feed-forward
is a routed set of small gated experts.
"""

from __future__ import annotations

import math

import torch


def layer_norm(x, weight, eps):
    mean = x.mean(dim=-1, keepdim=True)
    centred = x - mean
    variance = (centred * centred).mean(dim=-1, keepdim=True)
    return centred / torch.sqrt(variance + eps) * weight


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def key_frequencies(rot) -> tuple[list[float], float]:
    """Frequencies of the dims/2 pairs of the query/key rotation and the factor on sine and cosine.
    Without ``scaling`` pair i has base^(-2i/dims) and the factor is 1.  With it, pairs whose
    wavelength is long against the original context are slowed by ``factor``, short ones are left
    alone, and a linear ramp over the pair index joins the two."""
    base, dims = float(rot["base"]), int(rot["dims"])
    plain = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if not scaling:
        return plain, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    low = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    high = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(plain):
        ramp = min(max((i - low) / max(high - low, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def turn(vector, positions, frequencies, magnitude=1.0, sign=1.0):
    """Pairs (2i, 2i + 1) of the last axis, i < len(frequencies), turned by sign * position *
    frequencies[i]; sine and cosine times ``magnitude``; the other entries pass.  vector [T, ..., n]."""
    out = vector.clone()
    shape = (-1,) + (1,) * (vector.dim() - 2)
    for i, f in enumerate(frequencies):
        angle = positions.to(vector.dtype) * f * sign
        cos = (torch.cos(angle) * magnitude).reshape(shape)
        sin = (torch.sin(angle) * magnitude).reshape(shape)
        u, v = vector[..., 2 * i], vector[..., 2 * i + 1]
        out[..., 2 * i] = u * cos - v * sin
        out[..., 2 * i + 1] = v * cos + u * sin
    return out


def value_frequencies(base: float, vdim: int) -> list[float]:
    return [base ** (-2.0 * m / vdim) for m in range(vdim // 2)]


def attention(h, t, prefix, mixer, eps):
    heads, groups, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    length = h.shape[0]
    positions = torch.arange(length)
    # norms over the whole projections, before the split into heads
    q = rms(h @ t[prefix + "q"].T, eps) * t[prefix + "q.norm"]
    k = rms(h @ t[prefix + "k"].T, eps) * t[prefix + "k.norm"]
    v = (h @ t[prefix + "v"].T).reshape(length, groups, vdim)
    frequencies, magnitude = key_frequencies(mixer["rot"])
    q = turn(q.reshape(length, heads, dim), positions, frequencies, magnitude)
    k = turn(k.reshape(length, groups, dim), positions, frequencies, magnitude)
    around = value_frequencies(float(mixer["rot"]["base"]), vdim)
    v = turn(rms(v, eps), positions, around)
    out = torch.zeros(length, heads, vdim, dtype=h.dtype)
    per_group = heads // groups
    for head in range(heads):
        g = head // per_group
        scores = (q[:, head] @ k[:, g].T) * mixer["scale"]
        for i in range(length):
            weights = torch.softmax(scores[i, : i + 1], dim=0)
            out[i, head] = weights @ v[: i + 1, g]
    out = turn(out, positions, around, sign=-1.0)
    return out.reshape(length, heads * vdim) @ t[prefix + "o"].T


CLOSE_CALL = 0.02


def route(h, t, prefix, router, risk_out=None):
    """Per token: the chosen experts (indices) and their weights.  ``risk_out`` (a list) receives, per
    token, how much weight hangs on a close call: where the last chosen and the first left-out choice
    score (or the last kept and the first dropped group) lie within CLOSE_CALL of each other, the
    larger of the two experts' scores, else 0.  Tests of reduced precision leave such tokens out."""
    experts, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    scores = torch.softmax(h @ t[prefix + "router"].T, dim=-1)           # [T, experts]
    choice = scores + t[prefix + "correction"]
    size = experts // count
    best = choice.reshape(-1, count, size).max(dim=-1).values           # [T, count]
    kept = best.topk(keep, dim=-1).indices
    allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
    allowed = allowed.repeat_interleave(size, dim=1)
    choice = torch.where(allowed, choice, torch.full_like(choice, -math.inf))
    chosen = choice.topk(top, dim=-1).indices
    if risk_out is not None:
        risk = torch.zeros(h.shape[0], dtype=h.dtype)
        if top < experts:
            ranked = choice.topk(top + 1, dim=-1)
            close = (ranked.values[:, top - 1] - ranked.values[:, top]) < CLOSE_CALL
            risk = torch.where(close, scores.gather(1, ranked.indices[:, top - 1:top + 1]).max(dim=-1).values, risk)
        if keep < count:
            ranked = best.topk(keep + 1, dim=-1)
            close = (ranked.values[:, keep - 1] - ranked.values[:, keep]) < CLOSE_CALL
            pair = scores.reshape(-1, count, size).max(dim=-1).values.gather(1, ranked.indices[:, keep - 1:keep + 1])
            risk = torch.maximum(risk, torch.where(close, pair.max(dim=-1).values, torch.zeros_like(risk)))
        risk_out.append(risk)
    return chosen, scores.gather(1, chosen)


def experts(h, t, prefix, mlp, risk_out=None):
    chosen, weights = route(h, t, prefix, mlp["router"], risk_out)
    out = torch.zeros_like(h)
    for token in range(h.shape[0]):
        for e, w in zip(chosen[token].tolist(), weights[token]):
            gate = h[token] @ t[f"{prefix}e{e}.gate"].T
            up = h[token] @ t[f"{prefix}e{e}.up"].T
            out[token] += w * ((gate * torch.sigmoid(gate) * up) @ t[f"{prefix}e{e}.down"].T)
    return out


def forward(config, tensors, tokens, dtype=torch.float64, layers_out=None, risk_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the stream after
    every layer, ``risk_out`` (a list) one tensor per routed layer (see ``route``)."""
    t = {name: (value.to(dtype) if value.is_floating_point() else value) for name, value in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(config["embedding"]["scale"])
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        if layer["type"] != "attention":
            raise ValueError(layer["type"])
        mixed = attention(layer_norm(x, t[p + "norm1"], eps), t, p + "mix.", layer["mixer"], eps)
        x = x + layer_norm(mixed, t[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            passed = experts(layer_norm(x, t[p + "norm2"], eps), t, p + "mlp.", layer["mlp"], risk_out)
            x = x + layer_norm(passed, t[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, t["final.norm"], eps) @ t["head"].T
