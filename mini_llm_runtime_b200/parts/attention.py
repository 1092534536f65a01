"""Grouped-query causal self-attention over the paged cache.

q = x Wq^T + bq, k = x Wk^T + bk, v = x Wv^T + bv (one fused product on the concatenated
weights), position encoding on q and k, k and v stored to the cache, every row attends to its
request's cached keys (optionally only the last ``window`` of them) with query head h reading kv
head h // (heads / kv_heads), then o = attn Wo^T.  Reference: the ``_attention`` function of
src/mini_llm_runtime/qwen_model_runner.py:75-183 and the decode kernel
csrc/paged_attention_cuda.cu:25-106; the reference keeps q/k/v as three products and has no window.
"""

from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from ..ops import AttentionBatch
from .base import KVCacheNeed, Mixer, TensorSpec, build_part, register_part


class GQAAttention(Mixer):
    graph_safe = True
    supports_norm_fusion = True
    plan_key = "paged_attention"     # every attention layer of a model reads the same work lists

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.num_heads = int(a["num_heads"])
        self.num_kv_heads = int(a["num_kv_heads"])
        self.head_dim = int(a["head_dim"])
        self.qkv_bias = bool(a.get("qkv_bias", False))
        self.out_bias = bool(a.get("out_bias", False))
        self.window = a.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be divisible by num_kv_heads")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("an attention window must be positive")
        self.scale = float(self.head_dim) ** -0.5
        # the position encoding is optional: without one, q and k are used as projected
        self.position = build_part("position", a["position"], compute_dtype) if a.get("position") else None
        self._no_rotation: torch.Tensor | None = None
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None
        self.input_norm_eps: float | None = None     # set once the preceding norm's weight is folded in

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, None if self.window is None else int(self.window))

    def tensors(self):
        q_rows = self.num_heads * self.head_dim
        kv_rows = self.num_kv_heads * self.head_dim
        p = self.prefix
        out = {
            p + "q_proj.weight": TensorSpec((q_rows, self.hidden_size)),
            p + "k_proj.weight": TensorSpec((kv_rows, self.hidden_size)),
            p + "v_proj.weight": TensorSpec((kv_rows, self.hidden_size)),
            p + "o_proj.weight": TensorSpec((self.hidden_size, q_rows)),
        }
        if self.qkv_bias:
            out[p + "q_proj.bias"] = TensorSpec((q_rows,), init="bias")
            out[p + "k_proj.bias"] = TensorSpec((kv_rows,), init="bias")
            out[p + "v_proj.bias"] = TensorSpec((kv_rows,), init="bias")
        if self.out_bias:
            out[p + "o_proj.bias"] = TensorSpec((self.hidden_size,), init="bias")
        return out

    def load(self, tensors, device):
        p = self.prefix
        # q, k and v rows stacked so that one product yields [q heads | k heads | v heads].
        self.w_qkv = self._to_compute(
            torch.cat([tensors[p + f"{n}_proj.weight"] for n in "qkv"], dim=0), device)
        if self.qkv_bias:
            self.b_qkv = self._to_compute(
                torch.cat([tensors[p + f"{n}_proj.bias"] for n in "qkv"], dim=0), device)
        self.w_o = self._to_compute(tensors[p + "o_proj.weight"], device)
        if self.out_bias:
            self.b_o = self._to_compute(tensors[p + "o_proj.bias"], device)
        if self.position is not None:
            self.position.load({}, device)
        else:
            self._no_rotation = torch.zeros(self.head_dim // 2, dtype=torch.float32, device=device)

    def absorb_input_norm(self, weight, eps):
        folded = self.w_qkv.float() * weight.to(self.w_qkv.device).float()[None, :]
        self.w_qkv = folded.to(self.compute_dtype).contiguous()
        self.input_norm_eps = float(eps)

    def step_plan(self, host):
        return ops.current().plan_attention(host.lengths, host.position_start)

    def _batch(self, ctx, view) -> AttentionBatch:
        """The step's ragged batch as the attention kernels want it; built once per step and cache
        group and shared by the layers of that group."""
        batch = view.shared.get("attention_batch")
        if batch is None:
            arrays, counts = ctx.plans.get(self.plan_key, ({}, {}))
            batch = AttentionBatch(
                seg_q_start=ctx.seg_q_start, seg_q_len=ctx.seg_q_len, seg_pos0=ctx.seg_pos0, seg_slot=ctx.seg_slot,
                block_table=view.block_table, num_segments=ctx.num_segments, max_q_len=ctx.max_q_len,
                max_kv_len=ctx.max_kv_len, plan=arrays, counts=counts)
            view.shared["attention_batch"] = batch
        return batch

    def forward(self, x, ctx, view, writes_cache, raw_input=False, residual=None):
        """``raw_input``: x is the un-normalised stream and the q/k/v product applies the row scale
        of the folded norm.  ``residual``: the output product adds into it in place."""
        k = ops.current()
        qkv = k.linear(x, self.w_qkv, self.b_qkv, rms_eps=self.input_norm_eps if raw_input else None)
        batch = self._batch(ctx, view)
        frequencies = self._no_rotation if self.position is None else self.position.rotary_frequencies()
        if frequencies is not None:
            # a plain rotary encoding (or none): rotation, cache write and attention may share kernels
            mixed = k.rope_paged_attention(qkv, ctx.positions, frequencies, view.slots, view.k_pool, view.v_pool,
                                           batch, self.num_heads, self.num_kv_heads, self.head_dim, self.scale,
                                           self.window, writes_cache)
        else:
            q = self.position.rotate_and_store(qkv, ctx, view, self.num_heads, self.num_kv_heads, self.head_dim,
                                               writes_cache)
            mixed = k.paged_attention(q, view.k_pool, view.v_pool, batch, self.num_heads, self.num_kv_heads,
                                      self.head_dim, self.scale, self.window)
        return k.linear(mixed, self.w_o, self.b_o, residual=residual)


class DifferentialAttention(Mixer):
    """Grouped-query attention with two softmax maps per head over shared values.

    q = Wq x holds, per head, [map 1 | map 2] (2 * dim numbers); k = Wk x likewise per kv head; v = Wv x
    has ``vdim`` numbers per kv head.  Every (head, map) of q and k is RMS-normalised over ``dim``
    with a weight shared by all heads and maps; positions do not enter the scores.  Position i sees
    key j if j <= i and (i - j < window or j < keep_first); window 0 means all earlier keys.  With
    a1, a2 the maps' outputs and lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (one number per
    layer): o = a1 - lambda a2, o / rms(o) * (1 - diff), then Wo.  Scores, softmax and norms are
    32-bit; the cache holds normalised keys (both maps side by side) and values."""

    graph_safe = True
    plan_key = "paged_attention"

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.heads = int(a["heads"])
        self.kv_heads = int(a.get("kv_heads", self.heads))
        self.dim = int(a["dim"])
        self.vdim = int(a["vdim"])
        self.scale = float(a["scale"])
        self.diff = float(a["diff"])
        self.window = int(a.get("window") or 0)
        self.keep_first = int(a.get("keep_first") or 0) if self.window else 0
        self.eps = float(a["eps"])
        if self.heads % self.kv_heads:
            raise ValueError("heads must be divisible by kv_heads")
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None
        self.lam = 0.0

    def cache_need(self):
        return KVCacheNeed(self.kv_heads, 2 * self.dim, self.window or None, value_dim=self.vdim,
                           keep_first=self.keep_first)

    def tensors(self):
        p, h = self.prefix, self.hidden_size
        out = {p + "q": TensorSpec((2 * self.heads * self.dim, h)), p + "k": TensorSpec((2 * self.kv_heads * self.dim, h)),
               p + "v": TensorSpec((self.kv_heads * self.vdim, h)), p + "o": TensorSpec((h, self.heads * self.vdim)),
               p + "q.norm": TensorSpec((self.dim,), init="norm"), p + "k.norm": TensorSpec((self.dim,), init="norm")}
        for name in ("lq1", "lk1", "lq2", "lk2"):
            out[p + name] = TensorSpec((self.dim,), init="bias")
        return out

    def load(self, tensors, device):
        p = self.prefix
        self.w_qkv = self._to_compute(torch.cat([tensors[p + n] for n in "qkv"], dim=0), device)
        self.w_o = self._to_compute(tensors[p + "o"], device)
        self.q_norm = tensors[p + "q.norm"].to(device=device, dtype=torch.float32).contiguous()
        self.k_norm = tensors[p + "k.norm"].to(device=device, dtype=torch.float32).contiguous()
        l = {n: tensors[p + n].float() for n in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = float(torch.exp((l["lq1"] * l["lk1"]).sum()) - torch.exp((l["lq2"] * l["lk2"]).sum())) + self.diff

    def step_plan(self, host):
        return ops.current().plan_attention(host.lengths, host.position_start)

    def _batch(self, ctx, view) -> AttentionBatch:
        batch = view.shared.get("attention_batch")
        if batch is None:
            arrays, counts = ctx.plans.get(self.plan_key, ({}, {}))
            batch = AttentionBatch(
                seg_q_start=ctx.seg_q_start, seg_q_len=ctx.seg_q_len, seg_pos0=ctx.seg_pos0, seg_slot=ctx.seg_slot,
                block_table=view.block_table, num_segments=ctx.num_segments, max_q_len=ctx.max_q_len,
                max_kv_len=ctx.max_kv_len, plan=arrays, counts=counts)
            view.shared["attention_batch"] = batch
        return batch

    def forward(self, x, ctx, view, writes_cache):
        k = ops.current()
        qkv = k.linear(x, self.w_qkv, out_dtype=torch.float32)
        q = k.qk_norm_kv_write(qkv, self.q_norm, self.k_norm, self.eps, view.slots, view.k_pool, view.v_pool,
                               self.heads, self.kv_heads, self.dim, self.vdim, writes_cache)
        mixed = k.differential_attention(q, view.k_pool, view.v_pool, self._batch(ctx, view), self.heads,
                                         self.kv_heads, self.dim, self.vdim, self.scale, self.window,
                                         self.keep_first, self.lam, self.eps, 1.0 - self.diff)
        return k.linear(mixed, self.w_o, out_dtype=torch.float32)


class RotatedValueAttention(Mixer):
    """Grouped-query softmax attention over all earlier keys, with norms on q, k and v and a rotation
    of the values.

    q = Wq x [heads * dim], k = Wk x [kv_heads * dim], v = Wv x [kv_heads * vdim], no biases (one
    fused product).  With ``qk_norm="projection"`` q and k are RMS-normalised over the whole projection
    (all heads at once) with one learned weight per entry (``q.norm``, ``k.norm``); ``"none"`` leaves
    them.  Then the first ``rope_dims`` entries of every q and k head are turned by the position
    (``rope_layout`` ``interleaved``: pairs (2i, 2i + 1), ``half``: (i, i + rope_dims/2); base
    ``rope_base``; ``rope_scaling`` optional, see ``PairedRope``).  ``value_norm``: every value head is
    divided by its root mean square over vdim (no weight).  ``value_rotation``: the value of position j
    is turned by j over all vdim entries (same pair layout, base ``rope_base``, never scaled) before
    it is cached, and each head's output at position i is turned back by -i, so that the output
    depends on the distances i - j only.  score = (q . k) * ``scale``; query head h reads kv head
    h // (heads / kv_heads); Wo on the concatenated heads.

    32-bit: the norms, angles and rotations, scores and softmax; the projections leave 32-bit rows.
    In bfloat16 the products' operands, q, and the cached keys and values are bfloat16."""

    graph_safe = True
    plan_key = "paged_attention"

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.heads = int(a["heads"])
        self.kv_heads = int(a.get("kv_heads", self.heads))
        self.dim = int(a["dim"])
        self.vdim = int(a.get("vdim", self.dim))
        self.scale = float(a["scale"])
        self.eps = float(a["eps"])
        self.qk_norm = str(a.get("qk_norm", "projection"))
        if self.qk_norm not in ("projection", "none"):
            raise ValueError(f"unknown q/k norm {self.qk_norm!r}; known: projection, none")
        self.value_norm = bool(a.get("value_norm", True))
        self.value_rotation = bool(a.get("value_rotation", True))
        if self.heads % self.kv_heads:
            raise ValueError("heads must be divisible by kv_heads")
        layout = str(a.get("rope_layout", "interleaved"))
        rope_dims = int(a.get("rope_dims", self.dim))
        if rope_dims % 2 or not 0 < rope_dims <= self.dim:
            raise ValueError("the rotation covers an even number of entries, at most dim")
        self.position = build_part("position", PartSpec("rope_pairs", {
            "head_dim": rope_dims, "theta": float(a["rope_base"]), "layout": layout,
            "scaling": dict(a.get("rope_scaling") or {})}), compute_dtype)
        self.value_position = None
        if self.value_rotation:
            if self.vdim % 2:
                raise ValueError("values are turned in pairs: vdim must be even")
            self.value_position = build_part("position", PartSpec("rope_pairs", {
                "head_dim": self.vdim, "theta": float(a["rope_base"]), "layout": layout}), compute_dtype)
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    def cache_need(self):
        return KVCacheNeed(self.kv_heads, self.dim, None, value_dim=None if self.vdim == self.dim else self.vdim)

    def tensors(self):
        p, h = self.prefix, self.hidden_size
        out = {p + "q": TensorSpec((self.heads * self.dim, h)), p + "k": TensorSpec((self.kv_heads * self.dim, h)),
               p + "v": TensorSpec((self.kv_heads * self.vdim, h)), p + "o": TensorSpec((h, self.heads * self.vdim))}
        if self.qk_norm == "projection":
            out[p + "q.norm"] = TensorSpec((self.heads * self.dim,), init="norm")
            out[p + "k.norm"] = TensorSpec((self.kv_heads * self.dim,), init="norm")
        return out

    def load(self, tensors, device):
        p = self.prefix
        self.w_qkv = self._to_compute(torch.cat([tensors[p + n] for n in "qkv"], dim=0), device)
        self.w_o = self._to_compute(tensors[p + "o"], device)
        if self.qk_norm == "projection":
            self.q_norm = tensors[p + "q.norm"].to(device=device, dtype=torch.float32).contiguous()
            self.k_norm = tensors[p + "k.norm"].to(device=device, dtype=torch.float32).contiguous()
        self.position.load({}, device)
        if self.value_position is not None:
            self.value_position.load({}, device)

    def step_plan(self, host):
        return ops.current().plan_attention(host.lengths, host.position_start)

    def _batch(self, ctx, view) -> AttentionBatch:
        batch = view.shared.get("attention_batch")
        if batch is None:
            arrays, counts = ctx.plans.get(self.plan_key, ({}, {}))
            batch = AttentionBatch(
                seg_q_start=ctx.seg_q_start, seg_q_len=ctx.seg_q_len, seg_pos0=ctx.seg_pos0, seg_slot=ctx.seg_slot,
                block_table=view.block_table, num_segments=ctx.num_segments, max_q_len=ctx.max_q_len,
                max_kv_len=ctx.max_kv_len, plan=arrays, counts=counts)
            view.shared["attention_batch"] = batch
        return batch

    def forward(self, x, ctx, view, writes_cache):
        k = ops.current()
        interleaved = self.position.interleaved
        value_freq = None if self.value_position is None else self.value_position.rotary_frequencies()
        qkv = k.linear(x, self.w_qkv, out_dtype=torch.float32)
        q = k.rotated_prepare(qkv, ctx.positions, self.q_norm, self.k_norm, self.eps,
                              self.position.rotary_frequencies(), self.position.magnitude, value_freq, interleaved,
                              self.value_norm, view.slots, view.k_pool, view.v_pool, self.heads, self.kv_heads,
                              self.dim, self.vdim, writes_cache)
        mixed = k.paged_attention(q, view.k_pool, view.v_pool, self._batch(ctx, view), self.heads, self.kv_heads,
                                  self.dim, self.scale, None, value_dim=self.vdim)
        if value_freq is not None:
            mixed = k.turn_heads(mixed, ctx.positions, value_freq, self.heads, self.vdim, interleaved, sign=-1.0)
        return k.linear(mixed, self.w_o, out_dtype=torch.float32)


class HeadNormAttention(Mixer):
    """Grouped-query causal attention without a rotation, with q and k RMS-normalised per head.

    q = Wq x + bq [heads * dim], k = Wk x + bk [kv_heads * dim], v = Wv x + bv [kv_heads * vdim] (one fused
    product; ``bias=False``: no biases).  Every q and k head is divided by its root mean square over
    ``dim`` (eps inside the root) and, with ``qk_norm_weight``, multiplied by a learned weight [dim] shared
    by all heads (``q.norm``, ``k.norm``).  score = (q . k) * ``scale``; query head h reads key/value head
    h // (heads / kv_heads); every j <= i is visible.  ``weights`` chooses what becomes of the scores:

    * ``softmax``: the ordinary softmax over the visible keys;
    * ``sigmoid``: w = sigmoid(score + b_h) for every visible key, not normalised over the keys.  The
      optional pieces: ``distance_bias`` takes r1_h ln(1 + r2_h (i - j)) off the score (tensors ``r1``,
      ``r2`` [heads]); ``score_bias`` is b (tensor ``pb`` [heads]); ``head_mix`` mixes the weights across
      heads, w'_h = sum_g T[h, g] w_g (tensor ``talk`` [heads, heads]), before head h applies them to the
      values of its own key/value head.

    ``value_mix``: ``source`` hands this layer's values (as projected, 32-bit) to later layers of the same
    step under the name ``value_mix_key``; ``blend`` replaces its own by (1 - m) v + m * those, m being the
    tensor ``vmix`` (one number), before they are cached.  (A source layer's checkpoint carries ``vmix``
    too; it is not used.)  Wo on the concatenated heads; the result leaves in 32-bit floats.

    32-bit: the projections' results, the norms, the blend, scores and weights.  In bfloat16 the products'
    operands, q, and the cached keys and values are bfloat16."""

    graph_safe = True
    plan_key = "paged_attention"

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.heads = int(a["heads"])
        self.kv_heads = int(a.get("kv_heads", self.heads))
        self.dim = int(a["dim"])
        self.vdim = int(a.get("vdim", self.dim))
        self.scale = float(a["scale"])
        self.eps = float(a["eps"])
        self.bias = bool(a.get("bias", True))
        self.qk_norm_weight = bool(a.get("qk_norm_weight", False))
        self.weights = str(a.get("weights", "softmax"))
        if self.weights not in ("softmax", "sigmoid"):
            raise ValueError(f"unknown attention weights {self.weights!r}; known: softmax, sigmoid")
        self.distance_bias = bool(a.get("distance_bias", False))
        self.score_bias = bool(a.get("score_bias", False))
        self.head_mix = bool(a.get("head_mix", False))
        if self.weights == "softmax" and (self.distance_bias or self.score_bias or self.head_mix):
            raise ValueError("distance bias, score bias and head mixing belong to sigmoid weights")
        self.value_mix = a.get("value_mix")
        if self.value_mix not in (None, "source", "blend"):
            raise ValueError(f"unknown value_mix {self.value_mix!r}; known: source, blend")
        self.value_mix_key = str(a.get("value_mix_key", "first_values"))
        if self.heads % self.kv_heads:
            raise ValueError("heads must be divisible by kv_heads")
        self.w_qkv = self.b_qkv = self.w_o = self.q_norm = self.k_norm = None
        self.r1 = self.r2 = self.pb = self.talk = self.mix = None

    def cache_need(self):
        return KVCacheNeed(self.kv_heads, self.dim, None, value_dim=None if self.vdim == self.dim else self.vdim)

    def tensors(self):
        p, h = self.prefix, self.hidden_size
        sizes = {"q": self.heads * self.dim, "k": self.kv_heads * self.dim, "v": self.kv_heads * self.vdim}
        out = {p + name: TensorSpec((rows, h)) for name, rows in sizes.items()}
        if self.bias:
            out.update({p + name + ".b": TensorSpec((rows,), init="bias") for name, rows in sizes.items()})
        out[p + "o"] = TensorSpec((h, self.heads * self.vdim))
        if self.qk_norm_weight:
            out[p + "q.norm"] = TensorSpec((self.dim,), init="norm")
            out[p + "k.norm"] = TensorSpec((self.dim,), init="norm")
        if self.distance_bias:
            out[p + "r1"] = TensorSpec((self.heads,), init="unit")
            out[p + "r2"] = TensorSpec((self.heads,), init="unit")
        if self.score_bias:
            out[p + "pb"] = TensorSpec((self.heads,), init="bias")
        if self.head_mix:
            out[p + "talk"] = TensorSpec((self.heads, self.heads), init="matrix")
        if self.value_mix is not None:
            out[p + "vmix"] = TensorSpec((), init="unit")
        return out

    def load(self, tensors, device):
        p = self.prefix

        def f32(name):
            return tensors[p + name].to(device=device, dtype=torch.float32).contiguous()

        self.w_qkv = self._to_compute(torch.cat([tensors[p + n] for n in "qkv"], dim=0), device)
        if self.bias:
            self.b_qkv = self._to_compute(torch.cat([tensors[p + n + ".b"] for n in "qkv"], dim=0), device)
        self.w_o = self._to_compute(tensors[p + "o"], device)
        if self.qk_norm_weight:
            self.q_norm, self.k_norm = f32("q.norm"), f32("k.norm")
        if self.distance_bias:
            self.r1, self.r2 = f32("r1"), f32("r2")
        if self.score_bias:
            self.pb = f32("pb")
        if self.head_mix:
            self.talk = f32("talk")
        if self.value_mix == "blend":
            self.mix = f32("vmix").reshape(1)

    def step_plan(self, host):
        return ops.current().plan_attention(host.lengths, host.position_start)

    def _batch(self, ctx, view) -> AttentionBatch:
        batch = view.shared.get("attention_batch")
        if batch is None:
            arrays, counts = ctx.plans.get(self.plan_key, ({}, {}))
            batch = AttentionBatch(
                seg_q_start=ctx.seg_q_start, seg_q_len=ctx.seg_q_len, seg_pos0=ctx.seg_pos0, seg_slot=ctx.seg_slot,
                block_table=view.block_table, num_segments=ctx.num_segments, max_q_len=ctx.max_q_len,
                max_kv_len=ctx.max_kv_len, plan=arrays, counts=counts)
            view.shared["attention_batch"] = batch
        return batch

    def forward(self, x, ctx, view, writes_cache):
        k = ops.current()
        qkv = k.linear(x, self.w_qkv, self.b_qkv, out_dtype=torch.float32)
        other = None
        if self.value_mix == "source":
            ctx.shared[self.value_mix_key] = qkv[:, (self.heads + self.kv_heads) * self.dim:]
        elif self.value_mix == "blend":
            other = ctx.shared.get(self.value_mix_key)
            if other is None:
                raise ValueError(f"no earlier layer of this step handed out {self.value_mix_key!r}")
        q = k.head_norm_kv_write(qkv, self.q_norm, self.k_norm, self.eps, view.slots, view.k_pool, view.v_pool,
                                 self.heads, self.kv_heads, self.dim, self.vdim, writes_cache, other_values=other,
                                 mix=self.mix)
        batch = self._batch(ctx, view)
        if self.weights == "softmax":
            mixed = k.paged_attention(q, view.k_pool, view.v_pool, batch, self.heads, self.kv_heads, self.dim,
                                      self.scale, None, value_dim=self.vdim)
        else:
            mixed = k.sigmoid_attention(q, view.k_pool, view.v_pool, batch, self.heads, self.kv_heads, self.dim,
                                        self.vdim, self.scale,
                                        distance=(self.r1, self.r2) if self.distance_bias else None,
                                        score_bias=self.pb, head_mix=self.talk)
        return k.linear(mixed, self.w_o, out_dtype=torch.float32)


register_part("mixer", "gqa_attention", GQAAttention)
register_part("mixer", "head_norm_attention", HeadNormAttention)
register_part("mixer", "differential_attention", DifferentialAttention)
register_part("mixer", "rotated_value_attention", RotatedValueAttention)
