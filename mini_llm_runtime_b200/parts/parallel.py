"""Several mixers side by side in one layer.

All branches read the same input rows; each branch's output is RMS-normalised over the model width
(eps inside the root) with a plain learned weight of its own, and the layer's mixer output is
``factor`` times their sum (the mean, for ``factor`` = 1 / branches).  A branch is any registered
mixer, named by a ``PartSpec``; the branches' cache needs (keys and values of one, fixed-size states
of another) together form the layer's cache entry, and the branches see the same cache view.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, TensorSpec, build_part, register_part


class ParallelMixers(Mixer):
    """``branches``: a tuple of (name, PartSpec of a mixer, checkpoint name of its output weight [hidden]).
    At most one branch may keep keys and values, and state names must differ between branches (the
    cache manager checks both).  Two branches are fused into one kernel (both norms, the weights and the
    mean); the result is 32-bit rows."""

    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.eps = float(a["eps"])
        self.branches = [(str(name), build_part("mixer", part_spec, compute_dtype), str(weight))
                         for name, part_spec, weight in a["branches"]]
        if len(self.branches) != 2:
            raise ValueError("a parallel layer has two branches")
        self.factor = float(a.get("factor", 1.0 / len(self.branches)))
        self.graph_safe = all(branch.graph_safe for _, branch, _ in self.branches)
        keys = {branch.plan_key for _, branch, _ in self.branches if branch.plan_key is not None}
        if len(keys) > 1:
            raise ValueError(f"the branches name different work lists: {sorted(keys)}")
        self.plan_key = next(iter(keys), None)
        self.out_weights: list[torch.Tensor] = []

    def cache_need(self):
        needs = []
        for _, branch, _ in self.branches:
            need = branch.cache_need()
            if need is not None:
                needs.extend(need if isinstance(need, (tuple, list)) else (need,))
        return tuple(needs) if needs else None

    def tensors(self):
        out = {}
        for _, branch, weight in self.branches:
            out.update(branch.tensors())
            out[weight] = TensorSpec((self.hidden_size,), init="norm")
        return out

    def load(self, tensors, device):
        self.out_weights = []
        for _, branch, weight in self.branches:
            branch.load(tensors, device)
            self.out_weights.append(tensors[weight].to(device=device, dtype=torch.float32).contiguous())

    def step_plan(self, host):
        for _, branch, _ in self.branches:
            if branch.plan_key is not None:
                return branch.step_plan(host)
        return {}, {}

    def forward(self, x, ctx, view, writes_cache):
        outputs = [branch.forward(x, ctx, view, writes_cache) for _, branch, _ in self.branches]
        return ops.current().normed_mean(outputs[0], self.out_weights[0], outputs[1], self.out_weights[1], self.eps,
                                         self.factor)


register_part("mixer", "parallel_mixers", ParallelMixers)
