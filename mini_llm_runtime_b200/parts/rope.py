"""Rotate-half rotary position encoding (reference: src/mini_llm_runtime/qwen_model_runner.py:34-61).

inv_freq[i] = 1 / theta^(2i/D) for i < D/2 in float32; angle = position * inv_freq[i]; element i is
paired with element i + D/2; q and k are rotated, v is not.  The frequency table is computed once
here, with the reference's expression, and handed to the kernel, which evaluates sine and cosine
in float32 and fuses the rotation with the write of k and v into the cache pages.  No table over
positions is kept, so ``max_position_embeddings`` only bounds lengths, as in the reference.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import PositionEncoding, register_part


class RotateHalfRope(PositionEncoding):
    graph_safe = True
    interleaved = False      # pair i is (i, i + head_dim/2)

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.head_dim = int(self.args["head_dim"])
        self.theta = float(self.args["theta"])
        if self.head_dim % 2:
            raise ValueError("rotate-half position encoding needs an even head_dim")
        self._inv_freq_cpu = self._frequencies()
        self.inv_freq: torch.Tensor | None = None

    def _frequencies(self) -> torch.Tensor:
        exponents = torch.arange(0, self.head_dim, 2, dtype=torch.float32) / self.head_dim
        return 1.0 / (self.theta ** exponents)

    def load(self, tensors, device):
        self.inv_freq = self._inv_freq_cpu.to(device)

    def rotate_and_store(self, qkv, ctx, view, num_heads, num_kv_heads, head_dim, write_kv):
        if head_dim != self.head_dim:
            raise ValueError(f"position encoding was built for head_dim {self.head_dim}, mixer has {head_dim}")
        return ops.current().rope_kv_write(qkv, ctx.positions, self.inv_freq, view.slots, view.k_pool,
                                           view.v_pool, num_heads, num_kv_heads, head_dim, write_kv)

    def rotary_frequencies(self):
        return self.inv_freq


class PairedRope(RotateHalfRope):
    """The same rotation for mixers that turn a vector of ``head_dim`` numbers themselves (their
    kernels take ``rotary_frequencies()`` and ``interleaved``): pair i is (i, i + head_dim/2), or, with
    ``layout="interleaved"``, (2i, 2i + 1); it turns by position * theta^(-2i/head_dim).  The frequencies
    are evaluated in 64-bit and rounded once.

    ``scaling`` = {factor, original, fast, slow} stretches the long wavelengths for contexts beyond the
    ``original`` one: with pair(t) = head_dim * ln(original / (2 pi t)) / (2 ln theta) the index of the
    pair that makes t turns over the original context, low = max(floor(pair(fast)), 0), high =
    min(ceil(pair(slow)), head_dim - 1) and ramp_i = clamp((i - low) / max(high - low, 0.001), 0, 1), pair
    i gets f_i / factor * ramp_i + f_i * (1 - ramp_i); ``magnitude`` = 0.1 ln(factor) + 1 multiplies
    sine and cosine (1 without scaling)."""

    def __init__(self, spec, compute_dtype):
        layout = str(spec.args.get("layout", "half"))
        if layout not in ("half", "interleaved"):
            raise ValueError(f"unknown pair layout {layout!r}; known: half, interleaved")
        scaling = dict(spec.args.get("scaling") or {})
        if scaling and any(name not in scaling for name in ("factor", "original", "fast", "slow")):
            raise ValueError("a frequency scaling needs factor, original, fast and slow")
        self.scaling = scaling
        self.magnitude = 0.1 * math.log(float(scaling["factor"])) + 1.0 if scaling else 1.0
        super().__init__(spec, compute_dtype)
        self.interleaved = layout == "interleaved"

    def _frequencies(self):
        n = self.head_dim
        exponents = torch.arange(0, n, 2, dtype=torch.float64) / n
        plain = self.theta ** -exponents
        if not self.scaling:
            return plain.to(torch.float32)
        factor, original = float(self.scaling["factor"]), float(self.scaling["original"])

        def pair_of(turns: float) -> float:
            return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        low = max(math.floor(pair_of(float(self.scaling["fast"]))), 0)
        high = min(math.ceil(pair_of(float(self.scaling["slow"]))), n - 1)
        index = torch.arange(n // 2, dtype=torch.float64)
        ramp = ((index - low) / max(high - low, 0.001)).clamp(0.0, 1.0)
        return (plain / factor * ramp + plain * (1.0 - ramp)).to(torch.float32)

    def rotate_and_store(self, qkv, ctx, view, num_heads, num_kv_heads, head_dim, write_kv):
        raise NotImplementedError("this encoding is applied by the mixer's own kernels")


register_part("position", "rope_half", RotateHalfRope)
register_part("position", "rope_pairs", PairedRope)
