"""RMSNorm: y = w * x * rsqrt(mean(x^2) + eps), all in float32, eps inside the root, no centering
and no bias (reference: src/mini_llm_runtime/qwen_model_runner.py:22-26).  The reference casts the
normalised row back to the model dtype before multiplying by w; here the product is taken in
float32 and rounded once."""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, TensorSpec, register_part


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.size = int(self.args["size"])
        self.eps = float(self.args["eps"])
        self.weight: torch.Tensor | None = None
        self.folded = False       # True once the weight lives in the matrix that follows

    def tensors(self):
        return {self.prefix + "weight": TensorSpec((self.size,), init="norm")}

    def load(self, tensors, device):
        self.weight = self._keep_precision(tensors[self.prefix + "weight"], device)

    def fold(self):
        self.folded = True
        return self.weight, self.eps

    def forward(self, x):
        return ops.current().rms_norm(x, None if self.folded else self.weight, self.eps)

    def add_forward(self, residual, delta):
        return ops.current().add_rms_norm(residual, delta, None if self.folded else self.weight, self.eps)


class ScalarRMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * g with a single learned number g for the whole row.  It reads
    a 32-bit residual stream and hands out rows in the compute dtype (``forward``), or both those and
    the 32-bit rows (``forward_both``) for what continues in 32-bit.  The checkpoint tensor (a scalar)
    is named by the spec (``tensor``)."""

    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.eps = float(self.args["eps"])
        self.tensor = self.args.get("tensor") or self.prefix + "weight"
        self.gain: torch.Tensor | None = None

    def tensors(self):
        return {self.tensor: TensorSpec((), init="norm")}

    def load(self, tensors, device):
        self.gain = tensors[self.tensor].to(device=device, dtype=torch.float32).reshape(1).contiguous()

    def forward(self, x):
        return ops.current().scalar_rms_norm(x, self.gain, self.eps, self.compute_dtype)

    def forward_both(self, x):
        return ops.current().scalar_rms_norm(x, self.gain, self.eps, self.compute_dtype, want_float=True)


class LayerNorm(Norm):
    """y = (x - mean) / sqrt(variance + eps) * w + b over each row, the variance being the mean of the
    squared deviations; statistics, weight and bias in 32-bit.  It reads 32-bit rows.  Three uses, all
    one pass of the same kernel over a 32-bit residual stream:

    * ``forward(x)``: the normalised rows in the compute dtype (the input of a sublayer);
    * ``add_into(stream, delta)``: stream += LN(delta), for a norm that sits behind a sublayer;
    * ``add_forward(stream, delta, post=, offset=)``: stream += delta (normalised by ``post`` first,
      if given), stream += offset (a vector, if given), then this norm of the new stream.

    The checkpoint names come from the spec: ``tensor`` (weight) and ``tensor`` + ".b" (bias), unless
    ``bias_tensor`` names it.  With ``bias=False`` the norm has a weight only: the checkpoint holds no
    bias and the kernels get a vector of zeros (adding 0 changes no bit)."""

    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.size = int(self.args["size"])
        self.eps = float(self.args["eps"])
        self.tensor = self.args.get("tensor") or self.prefix + "weight"
        self.has_bias = bool(self.args.get("bias", True))
        self.bias_tensor = self.args.get("bias_tensor") or self.tensor + ".b"
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def tensors(self):
        out = {self.tensor: TensorSpec((self.size,), init="norm")}
        if self.has_bias:
            out[self.bias_tensor] = TensorSpec((self.size,), init="bias")
        return out

    def load(self, tensors, device):
        self.weight = tensors[self.tensor].to(device=device, dtype=torch.float32).contiguous()
        if self.has_bias:
            self.bias = tensors[self.bias_tensor].to(device=device, dtype=torch.float32).contiguous()
        else:
            self.bias = torch.zeros(self.size, dtype=torch.float32, device=device)

    @property
    def pair(self):
        return self.weight, self.bias

    def forward(self, x, offset=None):
        return ops.current().layer_norm_step(x, self.eps, offset=offset, norm=self.pair, out_dtype=self.compute_dtype)

    def add_into(self, stream, delta):
        ops.current().layer_norm_step(stream, self.eps, delta=delta, delta_norm=self.pair)
        return stream

    def add_forward(self, residual, delta, post=None, offset=None):
        if post is None:
            ops.current().add_residual(residual, delta)
            delta = None
        elif post.eps != self.eps:
            post.add_into(residual, delta)
            delta = None
        return ops.current().layer_norm_step(residual, self.eps, delta=delta,
                                             delta_norm=None if delta is None else post.pair, offset=offset,
                                             norm=self.pair, out_dtype=self.compute_dtype)


class StreamRMSNorm(Norm):
    """RMS norm for a 32-bit residual stream: y = v / sqrt(mean(v^2) + eps) * w, statistics and weight in
    32-bit.  With ``one_plus`` the checkpoint stores the weight's offset from one: w = 1 + stored.  The
    checkpoint name comes from the spec (``tensor``).  Uses, each one pass over the stream:

    * ``forward(x)``: the normalised rows in the compute dtype;
    * ``add_into(stream, delta)``: stream += norm(delta), for a norm that sits behind a sublayer;
    * ``add_cast(stream, delta)``: the same, and the new rows of the stream in the compute dtype (the input
      of a sublayer that reads the stream itself);
    * ``add_forward(stream, delta, post=)``: stream += post(delta) (``post`` another norm of this kind; the
      plain delta without one), then this norm of the new stream."""

    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.size = int(self.args["size"])
        self.eps = float(self.args["eps"])
        self.tensor = self.args.get("tensor") or self.prefix + "weight"
        self.one_plus = bool(self.args.get("one_plus", False))
        self.weight: torch.Tensor | None = None

    def tensors(self):
        return {self.tensor: TensorSpec((self.size,), init="bias" if self.one_plus else "norm")}

    def load(self, tensors, device):
        weight = tensors[self.tensor].to(device=device, dtype=torch.float32)
        self.weight = (1.0 + weight if self.one_plus else weight).contiguous()

    def forward(self, x):
        return ops.current().rms_norm_step(x, self.eps, norm_weight=self.weight, out_dtype=self.compute_dtype)

    def add_into(self, stream, delta):
        ops.current().rms_norm_step(stream, self.eps, delta=delta, delta_weight=self.weight)
        return stream

    def add_cast(self, stream, delta):
        if self.compute_dtype == torch.float32:
            return self.add_into(stream, delta)
        return ops.current().rms_norm_step(stream, self.eps, delta=delta, delta_weight=self.weight,
                                           out_dtype=self.compute_dtype)

    def add_forward(self, residual, delta, post=None):
        if post is None:
            ops.current().add_residual(residual, delta)
            return self.forward(residual)
        if post.eps != self.eps:
            post.add_into(residual, delta)
            return self.forward(residual)
        return ops.current().rms_norm_step(residual, self.eps, delta=delta, delta_weight=post.weight,
                                           norm_weight=self.weight, out_dtype=self.compute_dtype)


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "stream_rms_norm", StreamRMSNorm)
register_part("norm", "layer_norm", LayerNorm)
register_part("norm", "scalar_rms_norm", ScalarRMSNorm)
