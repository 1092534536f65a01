"""A plain, slow implementation of the ``Ratilorn`` design in float64 torch on the CPU: one function
per mechanism, whole sequences at once, no cache, no batching.  It shares no code with the package;
the tests compare the engine with it.

``config`` is the parsed config.json (a dict), ``tensors`` maps checkpoint names to tensors.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def _t(tensors, name):
    return tensors[name].to(F64)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def one_plus_norm(x, weight, eps):
    return rms(x, eps) * (1.0 + weight)


def silu(z):
    return z * torch.sigmoid(z)


def embed(tensors, tokens):
    positions = torch.arange(len(tokens))
    return _t(tensors, "embed")[torch.as_tensor(tokens)] + _t(tensors, "pos")[positions]


def sigmoid_attention(h, tensors, prefix, m, eps, v_first=None):
    """Per-head RMS-normalised q and k, score = q.k * scale - r1 ln(1 + r2 (i - j)), weight =
    sigmoid(score + pb) for j <= i (no normalisation over keys), weights mixed across heads by
    ``talk``, each head's mixed weights applied to the values of its own kv head.  Returns (output,
    the values that would be cached)."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ _t(tensors, prefix + "q").T + _t(tensors, prefix + "q.b")).view(T, H, D)
    k = (h @ _t(tensors, prefix + "k").T + _t(tensors, prefix + "k.b")).view(T, G, D)
    v = (h @ _t(tensors, prefix + "v").T + _t(tensors, prefix + "v.b")).view(T, G, V)
    if v_first is not None:
        lam = _t(tensors, prefix + "vmix")
        v = (1.0 - lam) * v + lam * v_first
    q, k = rms(q, eps), rms(k, eps)
    r1, r2, pb = _t(tensors, prefix + "r1"), _t(tensors, prefix + "r2"), _t(tensors, prefix + "pb")
    talk = _t(tensors, prefix + "talk")
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    distance = (i - j).clamp(min=0).to(F64)
    visible = (j <= i)
    weights = torch.zeros(H, T, T, dtype=F64)
    for head in range(H):
        kv = head // (H // G)
        score = (q[:, head] @ k[:, kv].T) * m["scale"] - r1[head] * torch.log1p(r2[head] * distance)
        weights[head] = torch.sigmoid(score + pb[head]) * visible
    mixed = torch.einsum("hg,gij->hij", talk, weights)
    out = torch.zeros(T, H, V, dtype=F64)
    for head in range(H):
        out[:, head] = mixed[head] @ v[:, head // (H // G)]
    return out.reshape(T, H * V) @ _t(tensors, prefix + "o").T, v


def softmax_attention(h, tensors, prefix, m, eps):
    """Grouped-query causal softmax attention; q and k RMS-normalised per head with a plain weight
    shared by all heads; positions do not enter."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ _t(tensors, prefix + "q").T + _t(tensors, prefix + "q.b")).view(T, H, D)
    k = (h @ _t(tensors, prefix + "k").T + _t(tensors, prefix + "k.b")).view(T, G, D)
    v = (h @ _t(tensors, prefix + "v").T + _t(tensors, prefix + "v.b")).view(T, G, V)
    q = rms(q, eps) * _t(tensors, prefix + "q.norm")
    k = rms(k, eps) * _t(tensors, prefix + "k.norm")
    mask = torch.full((T, T), -math.inf, dtype=F64).triu(1)
    out = torch.zeros(T, H, V, dtype=F64)
    for head in range(H):
        kv = head // (H // G)
        p = torch.softmax((q[:, head] @ k[:, kv].T) * m["scale"] + mask, dim=-1)
        out[:, head] = p @ v[:, kv]
    return out.reshape(T, H * V) @ _t(tensors, prefix + "o").T


def causal_conv_silu(u, weight, bias):
    """u [T, channels]; weight [channels, taps], the last column being the current token's; zeros
    before the start."""
    T, taps = u.shape[0], weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=F64), u])
    out = bias.expand(T, -1).clone()
    for tap in range(taps):
        out = out + padded[tap:tap + T] * weight[:, tap]
    return silu(out)


def state_space(h, tensors, prefix, m, eps):
    """Mamba-2: in-projection [z | x | B | C | dt], causal convolution and silu on x, B, C, scalar
    decay per head, S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T, y_t = S_t^T C_t + D x_t, gate by
    silu(z), RMS norm in groups, output projection."""
    T = h.shape[0]
    heads, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * P
    proj = h @ _t(tensors, prefix + "in").T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = causal_conv_silu(xbc, _t(tensors, prefix + "conv"), _t(tensors, prefix + "conv.b"))
    x = xbc[:, :inner].view(T, heads, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + _t(tensors, prefix + "dt_bias"))
    rate = torch.exp(_t(tensors, prefix + "A_log"))
    D = _t(tensors, prefix + "D")
    y = torch.zeros(T, heads, P, dtype=F64)
    for head in range(heads):
        g = head // (heads // G)
        S = torch.zeros(N, P, dtype=F64)
        for t in range(T):
            S = torch.exp(-rate[head] * dt[t, head]) * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + D[head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * _t(tensors, prefix + "norm")
    return y @ _t(tensors, prefix + "o").T


def parallel_mixer(h, tensors, prefix, m, eps):
    left = softmax_attention(h, tensors, prefix + "left.", m["left"], eps)
    right = state_space(h, tensors, prefix + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * _t(tensors, prefix + "left.out") + rms(right, eps) * _t(tensors, prefix + "right.out"))


def gated_ff(h, tensors, prefix):
    return (silu(h @ _t(tensors, prefix + "gate").T) * (h @ _t(tensors, prefix + "up").T)) @ _t(tensors, prefix + "down").T


def route(h, tensors, prefix, router):
    """(chosen experts [T, top], weights [T, top], margin): sigmoid scores, a correction that enters the
    choice only, groups ranked by the sum of their two best choice scores, weights renormalised.
    ``margin`` is the smallest gap between a chosen and an unchosen choice score (how close the
    closest call was)."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    s = torch.sigmoid(h @ _t(tensors, prefix + "router").T)
    c = s + _t(tensors, prefix + "correction")
    per = E // count
    grouped = c.view(-1, count, per)
    group_score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
    kept = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros(c.shape[0], count, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = torch.where(allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), c, torch.full_like(c, -math.inf))
    order = masked.sort(dim=-1, descending=True)
    chosen = order.indices[:, :top]
    margin = math.inf
    if top < E:
        margin = float((order.values[:, top - 1] - order.values[:, top]).min())
    if keep < count:
        ranked = group_score.sort(dim=-1, descending=True).values
        margin = min(margin, float((ranked[:, keep - 1] - ranked[:, keep]).min()))
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20), margin


def moe_ff(h, tensors, prefix, mlp):
    chosen, weights, _ = route(h, tensors, prefix, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            out[t] += w * gated_ff(h[t:t + 1], tensors, f"{prefix}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_ff(h, tensors, prefix + "shared.")
    return out


def forward(config, tensors, tokens):
    """(logits [T, vocab], residual stream after every layer [layers, T, width])."""
    eps = config["norm"]["eps"]
    x = embed(tensors, tokens)
    v_first = None
    stream = []
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        if layer["type"] == "attention":
            mixer = layer["mixer"]
            if mixer.get("v_mix"):
                mixed, v = sigmoid_attention(x, tensors, prefix + "mix.", mixer, eps, v_first)
                if v_first is None:
                    v_first = v
            else:
                mixed, _ = sigmoid_attention(x, tensors, prefix + "mix.", mixer, eps)
        elif layer["type"] == "parallel":
            mixed = parallel_mixer(x, tensors, prefix + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + one_plus_norm(mixed, _t(tensors, prefix + "norm1"), eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            passed = gated_ff(x, tensors, prefix + "mlp.") if mlp["kind"] == "dense" else moe_ff(x, tensors, prefix + "mlp.", mlp)
            x = x + one_plus_norm(passed, _t(tensors, prefix + "norm2"), eps)
        stream.append(x.clone())
    logits = one_plus_norm(x, _t(tensors, "final.norm"), eps) @ _t(tensors, "embed").T * config["logit_scale"]
    return logits, torch.stack(stream)
