"""Pre-norm residual arrangement: h = x + mixer(norm(x)); out = h + feed_forward(norm(h))
(reference: the ``_decoder_layer`` function, src/mini_llm_runtime/qwen_model_runner.py:199-218).

The residual stream and the newest output not yet added to it travel together, so that each
add is fused into the norm that follows it: one kernel reads and writes the stream once.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Block, PendingDelta, register_part


class PreNormResidual(Block):
    """In bfloat16, when both norms are of the "row scale times weight" kind and mixer and
    feed-forward can take it, each norm's weight is folded into the matrix that follows it at load
    time.  Steps of few rows (decode) then run without norm kernels: the products apply the row
    scale themselves and the products that end the mixer and the feed-forward add their result
    into the stream in place.  Steps of many rows keep the arrangement below, with norm kernels
    that only scale.  The float32 path keeps the reference's order of operations."""

    folded = False

    def finish_load(self, compute_dtype):
        if (compute_dtype == torch.bfloat16 and self.mixer.supports_norm_fusion
                and self.feed_forward.supports_norm_fusion):
            first, second = self.mixer_norm.fold(), self.feed_forward_norm.fold()
            if first is None or second is None:
                raise ValueError("a norm that cannot be folded must say so before it is asked to")
            self.mixer.absorb_input_norm(*first)
            self.feed_forward.absorb_input_norm(*second)
            self.folded = True

    def forward(self, residual, pending, ctx, view, writes_cache):
        kernels = ops.current()
        if self.folded and kernels.fuses_norm(residual.shape[0]):
            if pending is not None:
                residual = kernels.add_inplace(residual, pending)
            self.mixer.forward(residual, ctx, view, writes_cache, raw_input=True, residual=residual)
            self.feed_forward.forward(residual, ctx, raw_input=True, residual=residual)
            return residual, None
        if pending is None:
            normed = self.mixer_norm.forward(residual)
        else:
            normed = self.mixer_norm.add_forward(residual, pending)
        mixed = self.mixer.forward(normed, ctx, view, writes_cache)
        normed = self.feed_forward_norm.add_forward(residual, mixed)
        return residual, self.feed_forward.forward(normed, ctx)


class ParallelShifted(Block):
    """One norm, two readers: with h = norm(x) and s = shift(h) (the token shift named ``shift`` among
    the layer's further parts), x <- x + mixer(s) + feed_forward(h).  The stream x is 32-bit floats
    and both sublayers hand back 32-bit rows, so the sum is taken in 32-bit and rounded once.  A layer
    without a feed-forward adds the mixer's output alone.  The shift's carried row is a state of the
    layer beside whatever the mixer keeps."""

    def cache_need(self):
        own = self.mixer.cache_need()
        own = () if own is None else (tuple(own) if isinstance(own, (tuple, list)) else (own,))
        return (*own, self.extras["shift"].state_need())

    def forward(self, residual, pending, ctx, view, writes_cache):
        kernels = ops.current()
        if pending is not None:
            residual = kernels.add_residual(residual, pending)
        h32, h = self.mixer_norm.forward_both(residual)
        wants_float = getattr(self.mixer, "wants_float_input", False)
        shifted = self.extras["shift"].forward(h32, ctx, view, torch.float32 if wants_float else None)[0]
        mixed = self.mixer.forward(shifted, ctx, view, writes_cache)
        passed = None if self.feed_forward is None else self.feed_forward.forward(h, ctx)
        return kernels.add_residual(residual, mixed, passed), None


class SandwichNorm(Block):
    """A norm before and one behind each sublayer: x <- x + post1(mixer(pre1(x))), then
    x <- x + post2(ff(pre2(x))); a layer without a feed-forward ends after the first.  The two norms
    behind the sublayers are the layer's further parts ``mixer_post_norm`` and ``feed_forward_post_norm``.
    The stream x is 32-bit floats; the sublayers hand back 32-bit rows.  Each "add the normalised
    output, then norm for the next sublayer" is one pass over the stream: the last output of the
    layer travels on as a ``PendingDelta`` and is added by the next layer's first norm (or the
    model's final norm), together with a vector the run order may ask to be added before the layer."""

    takes_offset = True

    def forward(self, residual, pending, ctx, view, writes_cache, offset=None):
        kernels = ops.current()
        if pending is None:
            normed = self.mixer_norm.forward(residual, offset=offset)
        elif isinstance(pending, PendingDelta):
            normed = self.mixer_norm.add_forward(residual, pending.tensor, post=pending.norm, offset=offset)
        else:
            normed = self.mixer_norm.add_forward(residual, pending, offset=offset)
        mixed = self.mixer.forward(normed, ctx, view, writes_cache)
        if self.feed_forward is None:
            return residual, PendingDelta(mixed, self.extras["mixer_post_norm"])
        normed = self.feed_forward_norm.add_forward(residual, mixed, post=self.extras["mixer_post_norm"])
        passed = self.feed_forward.forward(normed, ctx)
        return residual, PendingDelta(passed, self.extras["feed_forward_post_norm"])


class PostNormResidual(Block):
    """Norms on the sublayers' outputs only: x <- x + norm1(mixer(x)), then x <- x + norm2(ff(x)); the
    sublayers read the stream x itself (its rows in the compute dtype).  ``mixer_norm`` and
    ``feed_forward_norm`` are those two norms (``StreamRMSNorm`` or any norm with ``add_into`` /
    ``add_cast``).  The stream is 32-bit floats and the sublayers hand back 32-bit rows.  Each "add the
    normalised output, hand the new stream to the next sublayer" is one pass over the stream: the layer's
    last output travels on as a ``PendingDelta`` and is added by the next layer (or the model's final
    norm).  A layer without a feed-forward ends after the first add."""

    def _enter(self, residual, pending):
        """Settle what the layer before left pending; returns the stream's rows in the compute dtype."""
        dtype = self.mixer.compute_dtype
        if isinstance(pending, PendingDelta) and pending.norm is not None and hasattr(pending.norm, "add_cast"):
            return pending.norm.add_cast(residual, pending.tensor)
        if pending is not None:
            if isinstance(pending, PendingDelta):
                if pending.norm is not None:
                    pending.norm.add_into(residual, pending.tensor)
                    pending = None
                else:
                    pending = pending.tensor
            if pending is not None:
                ops.current().add_residual(residual, pending)
        if dtype == torch.float32:
            return residual
        return ops.current().rms_norm_step(residual, 0.0, out_dtype=dtype)

    def forward(self, residual, pending, ctx, view, writes_cache):
        rows = self._enter(residual, pending)
        mixed = self.mixer.forward(rows, ctx, view, writes_cache)
        if self.feed_forward is None:
            return residual, PendingDelta(mixed, self.mixer_norm)
        rows = self.mixer_norm.add_cast(residual, mixed)
        passed = self.feed_forward.forward(rows, ctx)
        return residual, PendingDelta(passed, self.feed_forward_norm)


register_part("block", "pre_norm_residual", PreNormResidual)
register_part("block", "post_norm_residual", PostNormResidual)
register_part("block", "sandwich_norm", SandwichNorm)
register_part("block", "parallel_shifted", ParallelShifted)
