"""Mixers that carry a matrix-valued state per head instead of a key/value cache.

Both keep, per request and head, a state S [dim, vdim] of 32-bit floats that starts at zero and is
advanced token by token; what enters the recurrence beside the projections (decays, gates, norms)
is 32-bit.  Projections leave as 32-bit rows so that nothing is rounded on the way into the
recurrence; the mixer's output projection leaves 32-bit rows for a 32-bit residual stream.

``wkv``    time mixing with a data-dependent per-channel decay and a bonus for the current token:
           every projection reads its own blend of the input with the previous token's input
           (coefficients ``mu.*``); w_t = exp(-exp(W2 tanh(W1 x_w) + w0));
           o_t = (S + diag(u) k_t v_t^T)^T r_t;  S <- diag(w_t) S + k_t v_t^T;
           out = Wo (o / rms(o) * norm * silu(Wg x_g)).
``state_space``  a selective state-space layer with a scalar decay per head (Mamba-2, "state-space
           duality"), see ``StateSpaceMixer``.
``hgrn2``  gated linear attention whose forget gate also sets what is written:
           f_t = l + (1 - l) sigmoid(Wf x + b);  S <- diag(f_t) S + (1 - f_t) v_t^T;
           o_t = S^T silu(Wq x);  out = Wo (o / rms(o) * norm).
"""

from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import Mixer, StateNeed, TensorSpec, build_part, register_part


def _float(tensor, device):
    return tensor.to(device=device, dtype=torch.float32).contiguous()


class WKVMixer(Mixer):
    graph_safe = True
    wants_float_input = True       # its own blends are taken of 32-bit rows

    BLENDS = ("r", "k", "v", "g", "w")

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.heads = int(a["heads"])
        self.dim = int(a["dim"])
        self.eps = float(a["eps"])
        self.inner = self.heads * self.dim
        # the decay's bottleneck width is whatever the checkpoint's w1/w2 have; random weights use this
        self.default_rank = int(a.get("decay_rank") or max(16, self.hidden_size // 16))
        # the blends with the previous token's input: a token shift with five coefficient vectors
        self.blend = build_part("shift", PartSpec("token_shift", {
            "hidden_size": self.hidden_size, "state": "previous_input",
            "tensors": tuple(self.prefix + "mu." + name for name in self.BLENDS)}), compute_dtype)
        self.w = {}
        self.decay_bias = self.bonus = self.norm = None

    def cache_need(self):
        return (StateNeed((self.heads, self.dim, self.dim), torch.float32, "state"), self.blend.state_need())

    def tensors(self):
        p, h, n = self.prefix, self.hidden_size, self.inner
        out = {p + name: TensorSpec((n, h)) for name in ("r", "k", "v", "g")}
        out[p + "o"] = TensorSpec((h, n))
        out[p + "w0"] = TensorSpec((n,), init="bias")
        out[p + "u"] = TensorSpec((self.heads, self.dim), init="bias")
        out[p + "norm"] = TensorSpec((n,), init="norm")
        out[p + "w1"] = TensorSpec((self.default_rank, h), flexible=(0,))
        out[p + "w2"] = TensorSpec((n, self.default_rank), flexible=(1,))
        out.update(self.blend.tensors())
        return out

    def load(self, tensors, device):
        p = self.prefix
        if tensors[p + "w1"].shape[0] != tensors[p + "w2"].shape[1]:
            raise ValueError(f"{p}w1 and {p}w2 disagree on the decay's bottleneck width")
        for name in ("r", "k", "v", "g", "o", "w1", "w2"):
            self.w[name] = self._to_compute(tensors[p + name], device)
        self.decay_bias = _float(tensors[p + "w0"], device)
        self.bonus = _float(tensors[p + "u"], device).reshape(-1)
        self.norm = _float(tensors[p + "norm"], device)
        self.blend.load(tensors, device)

    def forward(self, x, ctx, view, writes_cache):
        k = ops.current()
        xr, xk, xv, xg, xw = self.blend.forward(x, ctx, view)
        f32 = torch.float32
        r = k.linear(xr, self.w["r"], out_dtype=f32)
        key = k.linear(xk, self.w["k"], out_dtype=f32)
        value = k.linear(xv, self.w["v"], out_dtype=f32)
        gate = k.linear(xg, self.w["g"], out_dtype=f32)
        decay = k.linear(k.tanh_(k.linear(xw, self.w["w1"])), self.w["w2"], out_dtype=f32)
        mixed = k.bonus_recurrence(r, key, value, decay, gate, self.decay_bias, self.bonus, self.norm, self.eps,
                                   view.states["state"], ctx, self.heads, self.dim, self.compute_dtype)
        return k.linear(mixed, self.w["o"], out_dtype=f32)


class HGRN2Mixer(Mixer):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.heads = int(a["heads"])
        self.dim = int(a["dim"])
        self.vdim = int(a["vdim"])
        self.eps = float(a["eps"])
        self.w_qfv = self.w_o = self.forget_bias = self.lower = self.norm = None

    def cache_need(self):
        return StateNeed((self.heads, self.dim, self.vdim), torch.float32, "state")

    def tensors(self):
        p, h, n = self.prefix, self.hidden_size, self.heads * self.dim
        return {p + "q": TensorSpec((n, h)), p + "f": TensorSpec((n, h)), p + "f.b": TensorSpec((n,), init="bias"),
                p + "lower": TensorSpec((n,), init="unit"), p + "v": TensorSpec((self.heads * self.vdim, h)),
                p + "norm": TensorSpec((self.vdim,), init="norm"), p + "o": TensorSpec((h, self.heads * self.vdim))}

    def load(self, tensors, device):
        p = self.prefix
        # one product yields [q | f | v]
        self.w_qfv = self._to_compute(torch.cat([tensors[p + "q"], tensors[p + "f"], tensors[p + "v"]], dim=0), device)
        self.w_o = self._to_compute(tensors[p + "o"], device)
        self.forget_bias = _float(tensors[p + "f.b"], device)
        self.lower = _float(tensors[p + "lower"], device)
        self.norm = _float(tensors[p + "norm"], device)

    def forward(self, x, ctx, view, writes_cache):
        k = ops.current()
        n = self.heads * self.dim
        qfv = k.linear(x, self.w_qfv, out_dtype=torch.float32)
        mixed = k.forget_gate_recurrence(qfv[:, :n], qfv[:, n:2 * n], qfv[:, 2 * n:], self.forget_bias, self.lower,
                                         self.norm, self.eps, view.states["state"], ctx, self.heads, self.dim,
                                         self.vdim, self.compute_dtype)
        return k.linear(mixed, self.w_o, out_dtype=torch.float32)


class StateSpaceMixer(Mixer):
    """Selective state-space layer with a scalar decay per head.

    With inner = heads * vdim, N = ``state`` and G = ``groups``, one product W_in x yields
    [z: inner | x: inner | B: G N | C: G N | dt: heads].  x, B and C together pass a causal convolution
    per channel (``conv`` [channels, taps], last column the current token's, bias ``conv.b``, zeros before
    the request's start) and silu.  dt <- softplus(dt + dt_bias).  Per head h, reading group
    h // (heads / G):  S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T  (S: N x vdim),
    y_t = S_t^T C_t + D_h x_t.  Then y * silu(z), an RMS norm in ``norm_groups`` equal parts (each by its
    own root mean square) times ``norm``, and W_o.

    Per request the layer carries S (32-bit, kept transposed: [heads, vdim, N]) and the convolution's
    last taps - 1 inputs.  Everything between the in-projection and W_o is 32-bit."""

    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.heads = int(a["heads"])
        self.vdim = int(a["vdim"])
        self.n = int(a["state"])
        self.groups = int(a.get("groups", 1))
        self.taps = int(a["conv"])
        self.norm_groups = int(a.get("norm_groups", 1))
        self.eps = float(a["eps"])
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n
        if self.heads % self.groups or self.inner % self.norm_groups or self.taps < 2:
            raise ValueError("heads must divide into the groups, the inner width into the norm's parts, and the "
                             "convolution needs at least two taps")
        self.w_in = self.w_o = self.conv = self.conv_bias = self.dt_bias = self.a_log = self.skip = self.norm = None

    def cache_need(self):
        return (StateNeed((self.heads, self.vdim, self.n), torch.float32, "state"),
                StateNeed((self.taps - 1, self.channels), torch.float32, "conv"))

    def tensors(self):
        p, h = self.prefix, self.hidden_size
        return {p + "in": TensorSpec((2 * self.inner + 2 * self.groups * self.n + self.heads, h)),
                p + "conv": TensorSpec((self.channels, self.taps), init="bias"),
                p + "conv.b": TensorSpec((self.channels,), init="bias"),
                p + "dt_bias": TensorSpec((self.heads,), init="bias"),
                p + "A_log": TensorSpec((self.heads,), init="bias"),
                p + "D": TensorSpec((self.heads,), init="norm"),
                p + "norm": TensorSpec((self.inner,), init="norm"),
                p + "o": TensorSpec((h, self.inner))}

    def load(self, tensors, device):
        p = self.prefix
        self.w_in = self._to_compute(tensors[p + "in"], device)
        self.w_o = self._to_compute(tensors[p + "o"], device)
        self.conv = _float(tensors[p + "conv"], device)
        self.conv_bias = _float(tensors[p + "conv.b"], device)
        self.dt_bias = _float(tensors[p + "dt_bias"], device)
        self.a_log = _float(tensors[p + "A_log"], device)
        self.skip = _float(tensors[p + "D"], device)
        self.norm = _float(tensors[p + "norm"], device)

    def forward(self, x, ctx, view, writes_cache):
        k = ops.current()
        inner, gn = self.inner, self.groups * self.n
        projected = k.linear(x, self.w_in, out_dtype=torch.float32)
        mixed = k.causal_conv(projected[:, inner:inner + self.channels], self.conv, self.conv_bias, view.states["conv"],
                              ctx, "silu")
        y = k.state_space_scan(mixed[:, :inner], mixed[:, inner:inner + gn], mixed[:, inner + gn:],
                               projected[:, inner + self.channels:], self.dt_bias, self.a_log, self.skip,
                               view.states["state"], ctx, self.heads, self.vdim, self.n, self.groups)
        gated = k.gated_group_norm(y, projected[:, :inner], self.norm, self.eps, self.norm_groups, self.compute_dtype)
        return k.linear(gated, self.w_o, out_dtype=torch.float32)


register_part("mixer", "wkv", WKVMixer)
register_part("mixer", "state_space", StateSpaceMixer)
register_part("mixer", "hgrn2", HGRN2Mixer)
