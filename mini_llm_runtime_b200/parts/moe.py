"""A routed set of small gated feed-forward experts (mixture of experts).

Per token, with h the input row:

    z = R h                                   router logits, 32-bit
    s = softmax(z)  (or sigmoid(z))           scores over all experts
    c = s + correction                        choice scores (the correction enters the choice only)
    experts form ``groups`` equal groups of neighbours; a group's score is the sum of its ``group_top``
    largest c (1, the default: its largest c); only experts of the best ``keep`` groups can be chosen
    (the others count as minus infinity)
    chosen = the ``top`` largest c
    out = sum over chosen e of s_e * down_e(act(gate_e h) * up_e h)       (s_e / (sum of the chosen s +
                                                                           ``renorm_eps``) if ``renormalise``)
    out += shared(h)                          with ``shared`` = the inner width of one more gated expert of the
                                              same form that every token uses (tensors ``shared.gate|up|down``)

Experts have no biases.  Checkpoint names after the prefix: ``router`` [experts, hidden], ``correction``
[experts] (``correction=False``: none), ``e<j>.gate``, ``e<j>.up`` [inner, hidden], ``e<j>.down`` [hidden,
inner].  The experts' matrices are stacked at load time: [experts, 2 * inner, hidden] with gate and up
rows interleaved in blocks like ``GatedMLP``'s, and [experts, hidden, inner].

32-bit: the router product, scores, choice and weights, and the weighted sum; the result leaves in
32-bit floats.  In bfloat16 the experts' products have bfloat16 operands.
"""

from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import FeedForward, TensorSpec, build_part, register_part


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.intermediate_size = int(a["intermediate_size"])
        self.experts = int(a["experts"])
        self.top = int(a["top"])
        self.groups = int(a.get("groups", 1))
        self.keep = int(a.get("keep", self.groups))
        self.activation = str(a.get("activation", "silu"))
        if self.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"unknown gate activation {self.activation!r}")
        self.scoring = str(a.get("scoring", "softmax"))
        if self.scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"unknown router scoring {self.scoring!r}; known: softmax, sigmoid")
        self.renormalise = bool(a.get("renormalise", False))
        self.renorm_eps = float(a.get("renorm_eps", 0.0))
        self.group_top = int(a.get("group_top", 1))
        if self.group_top < 1:
            raise ValueError("a group's score sums at least one choice score")
        self.shared = None
        if a.get("shared"):
            self.shared = build_part("feed_forward", PartSpec("gated_mlp", {
                "hidden_size": self.hidden_size, "intermediate_size": int(a["shared"]),
                "activation": self.activation, "names": ("gate", "up", "down")}, self.prefix + "shared."), compute_dtype)
        self.has_correction = bool(a.get("correction", True))
        if self.experts % self.groups or not 0 < self.keep <= self.groups:
            raise ValueError("experts must divide into the groups, of which 1..groups are kept")
        if not 0 < self.top <= self.keep * (self.experts // self.groups):
            raise ValueError("top exceeds the experts of the kept groups")
        self.router = self.correction = self.w_gate_up = self.w_down = None
        self.block = self.intermediate_size

    def tensors(self):
        p, h, f = self.prefix, self.hidden_size, self.intermediate_size
        out = {p + "router": TensorSpec((self.experts, h))}
        if self.has_correction:
            out[p + "correction"] = TensorSpec((self.experts,), init="bias")
        for e in range(self.experts):
            out[f"{p}e{e}.gate"] = TensorSpec((f, h))
            out[f"{p}e{e}.up"] = TensorSpec((f, h))
            out[f"{p}e{e}.down"] = TensorSpec((h, f))
        if self.shared is not None:
            out.update(self.shared.tensors())
        return out

    def load(self, tensors, device):
        p, h, f = self.prefix, self.hidden_size, self.intermediate_size
        self.router = tensors[p + "router"].to(device=device, dtype=torch.float32).contiguous()
        if self.has_correction:
            self.correction = tensors[p + "correction"].to(device=device, dtype=torch.float32).contiguous()
        self.block = 64 if f % 64 == 0 else f
        stacked = []
        for e in range(self.experts):
            gate, up = tensors[f"{p}e{e}.gate"], tensors[f"{p}e{e}.up"]
            stacked.append(torch.cat([gate.view(-1, self.block, h), up.view(-1, self.block, h)], dim=1).reshape(2 * f, h))
        self.w_gate_up = self._to_compute(torch.stack(stacked), device)
        self.w_down = self._to_compute(torch.stack([tensors[f"{p}e{e}.down"] for e in range(self.experts)]), device)
        if self.shared is not None:
            self.shared.load(tensors, device)

    def forward(self, x, ctx):
        k = ops.current()
        chosen, weights = k.route_experts(x, self.router, self.correction, self.top, self.groups, self.keep,
                                          self.scoring, self.renormalise, group_top=self.group_top,
                                          renorm_eps=self.renorm_eps)
        out = k.routed_experts(x, chosen, weights, self.w_gate_up, self.w_down, self.block, self.activation)
        if self.shared is not None:
            out = k.add_residual(out, self.shared.forward(x, ctx))
        return out


register_part("feed_forward", "routed_experts", RoutedExperts)
