"""Token embedding and the two heads.

Embedding is a row gather without scaling (reference: qwen_model_runner.py:263).  The tied head
multiplies by the embedding matrix as the reference always does (:289-290); the separate
``lm_head.weight`` has no counterpart there (the reference rejects untied checkpoints).  Logits
leave the head as float32.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, Head, TensorSpec, register_part


class TokenEmbedding(Embedding):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.vocab_size = int(self.args["vocab_size"])
        self.hidden_size = int(self.args["hidden_size"])
        # ``tensor``: the table's checkpoint name; ``rows="float32"``: hand out 32-bit rows (for a
        # model whose residual stream is 32-bit), the table itself stays in the compute dtype
        self.tensor = self.args.get("tensor") or self.prefix + "weight"
        self.float_rows = str(self.args.get("rows", "")) == "float32"
        # ``scale``: every row is multiplied by it (in 32-bit; only with 32-bit rows)
        self.scale = float(self.args.get("scale", 1.0))
        if self.scale != 1.0 and not self.float_rows:
            raise ValueError("a scaled embedding hands out 32-bit rows (rows=\"float32\")")
        self.weight: torch.Tensor | None = None

    def tensors(self):
        return {self.tensor: TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors, device):
        self.weight = self._to_compute(tensors[self.tensor], device)

    def forward(self, token_ids, positions=None):
        if self.float_rows:
            return ops.current().embedding_rows32(token_ids, self.weight, self.scale)
        return ops.current().embedding(token_ids, self.weight)


class TiedHead(Head):
    """logits = x E^T.  A checkpoint may still carry the head's own matrix; it must then equal the
    embedding's tensor, whose checkpoint name the spec gives as ``tied_to`` (reference rule:
    src/mini_llm_runtime/qwen_weights.py:113-119).  Without ``tied_to`` nothing is compared."""

    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.vocab_size = int(self.args["vocab_size"])
        self.hidden_size = int(self.args["hidden_size"])
        self.tied_to = self.args.get("tied_to")
        self.scale = float(self.args.get("scale", 1.0))      # logits are multiplied by it (in 32-bit)
        self.own_copy = bool(self.args.get("own_copy", True))   # False: the checkpoint never carries a copy

    def tensors(self):
        if not self.own_copy:
            return {}
        return {self.prefix + "weight": TensorSpec((self.vocab_size, self.hidden_size), optional=True)}

    def load(self, tensors, device):
        copy = tensors.get(self.prefix + "weight")
        original = tensors.get(self.tied_to) if self.tied_to else None
        if copy is not None and original is not None and not torch.equal(copy, original):
            raise ValueError(f"{self.prefix}weight is present but differs from {self.tied_to} "
                             "although tie_word_embeddings is true")

    def extra_inputs(self):
        return (self.tied_to,) if self.tied_to else ()

    def forward(self, x, embedding):
        logits = ops.current().linear(x, embedding.weight, None, out_dtype=torch.float32)
        return logits if self.scale == 1.0 else ops.current().scale_(logits, self.scale)


class LinearHead(Head):
    """logits = x H^T with the head's own matrix: ``<prefix>weight``, or the checkpoint name the
    spec gives as ``tensor``."""

    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.vocab_size = int(self.args["vocab_size"])
        self.hidden_size = int(self.args["hidden_size"])
        self.tensor = self.args.get("tensor") or self.prefix + "weight"
        self.weight: torch.Tensor | None = None

    def tensors(self):
        return {self.tensor: TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors, device):
        self.weight = self._to_compute(tensors[self.tensor], device)

    def forward(self, x, embedding):
        return ops.current().linear(x, self.weight, None, out_dtype=torch.float32)


class TokenPositionEmbedding(Embedding):
    """row = E[token] + P[position]: a learned vector per position, added unscaled.  The sum is
    taken and handed on in 32-bit floats (the model's residual stream is 32-bit), whatever the
    compute dtype.  Checkpoint names come from the spec (``token_tensor``, ``position_tensor``)."""

    graph_safe = True
    needs_positions = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.vocab_size = int(self.args["vocab_size"])
        self.hidden_size = int(self.args["hidden_size"])
        self.max_positions = int(self.args["max_positions"])
        self.token_tensor = self.args.get("token_tensor") or self.prefix + "weight"
        self.position_tensor = self.args.get("position_tensor") or self.prefix + "positions"
        self.weight: torch.Tensor | None = None
        self.positions: torch.Tensor | None = None

    def tensors(self):
        return {self.token_tensor: TensorSpec((self.vocab_size, self.hidden_size)),
                self.position_tensor: TensorSpec((self.max_positions, self.hidden_size))}

    def load(self, tensors, device):
        self.weight = self._to_compute(tensors[self.token_tensor], device)
        self.positions = self._to_compute(tensors[self.position_tensor], device)

    def forward(self, token_ids, positions=None):
        return ops.current().embedding_positions(token_ids, positions, self.weight, self.positions)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "token_position_embedding", TokenPositionEmbedding)
register_part("head", "tied_head", TiedHead)
register_part("head", "linear_head", LinearHead)
