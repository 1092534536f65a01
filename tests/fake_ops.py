"""Stand-in for the CUDA kernels, in plain torch on the CPU, with the kernels' exact calling
contracts.  Tests install it with ``ops.use(FakeOps())`` to exercise everything above the kernels
(parts, model, cache manager, step function, scheduler, replay program) on a machine without a
GPU, the way the reference's own tests replace its kernel by a Python oracle
(tests/test_engine.py:82-101 there).  It is test equipment only: the package never selects it, and
the GPU tests do not use it.
"""

from __future__ import annotations

import numpy as np
import torch

from mini_llm_runtime_b200.cache.slots import COUNTER, LAST_TOKEN, LENGTH, read_record


class FakeOps:
    name = "fake-cpu"
    error_code = 0      # tests set this to make the next device check fail

    def raise_if_device_error(self):
        if self.error_code:
            code, self.error_code = self.error_code, 0
            from mini_llm_runtime_b200.ops import KernelError
            raise KernelError(f"a kernel's bounded wait ran out (code {code}); the results of the "
                              "steps since the last check are invalid")

    # ---- resident tables and slot records
    def plan_attention(self, lengths, position_start):
        return {}, {}

    def scatter_rows(self, table, row_index, rows):
        table[row_index.long()] = rows

    def decode_prepare(self, seg_slot, slot_state, *, token_ids=None, positions=None, seg_pos0=None, table=None,
                       page_size=0, kv_slots=None):
        for i, slot in enumerate(seg_slot.tolist()):
            position = int(slot_state[slot, LENGTH])
            if token_ids is not None:
                token_ids[i] = int(slot_state[slot, LAST_TOKEN])
            if positions is not None:
                positions[i] = position
            if seg_pos0 is not None:
                seg_pos0[i] = position
            if kv_slots is not None:
                page = int(table[slot, position // page_size])
                kv_slots[i] = page * page_size + position % page_size if page >= 0 else -1

    def advance_slots(self, seg_slot, slot_state, seg_q_len=None, seg_pos0=None):
        for i, slot in enumerate(seg_slot.tolist()):
            grow = 1 if seg_q_len is None else int(seg_q_len[i])
            base = int(slot_state[slot, LENGTH]) if seg_pos0 is None else int(seg_pos0[i])
            slot_state[slot, LENGTH] = base + grow

    def sample_slots(self, logits, row_slot, slot_state, advance=False):
        from plain_qwen2 import temperature_sample, uniform_from_seed

        tokens = torch.empty(logits.shape[0], dtype=torch.int32)
        for row, slot in enumerate(row_slot.tolist()):
            record = read_record(slot_state[slot].numpy())
            if record["temperature"] <= 0:
                token = int(torch.argmax(logits[row]))
            else:
                u = uniform_from_seed(record["seed"], record["counter"])
                token = int(temperature_sample(logits[row], record["temperature"], u)[0])
            tokens[row] = token
            slot_state[slot, LAST_TOKEN] = token
            slot_state[slot, COUNTER] += 1
            if advance:
                slot_state[slot, LENGTH] += 1
        return tokens

    def embedding(self, ids, table):
        return table[ids.long()].clone()

    def gather_rows(self, x, rows):
        return x[rows.long()].clone()

    def rms_norm(self, x, weight, eps):
        x32 = x.float()
        out = x32 * torch.rsqrt((x32 * x32).mean(-1, keepdim=True) + eps)
        if weight is not None:
            out = weight.float() * out
        return out.to(x.dtype)

    def add_inplace(self, target, delta):
        target.copy_((target.float() + delta.float()).to(target.dtype))
        return target

    def fuses_norm(self, rows):
        return 0 < rows <= 16

    def add_rms_norm(self, residual, delta, weight, eps):
        residual.copy_((residual.float() + delta.float()).to(residual.dtype))
        return self.rms_norm(residual, weight, eps)

    def swiglu(self, gate_up, block=None):
        inner = gate_up.shape[1] // 2
        block = block or inner
        blocks = gate_up.float().view(gate_up.shape[0], inner // block, 2, block)
        gate, up = blocks[:, :, 0].reshape(-1, inner), blocks[:, :, 1].reshape(-1, inner)
        return (torch.nn.functional.silu(gate) * up).to(gate_up.dtype)

    def linear_swiglu(self, x, weight, block, rms_eps=None):
        return self.swiglu(self.linear(x, weight, rms_eps=rms_eps), block)

    def linear(self, x, weight, bias=None, out_dtype=None, rms_eps=None, residual=None):
        x32 = x.float()
        if rms_eps is not None:
            x32 = x32 * torch.rsqrt((x32 * x32).mean(-1, keepdim=True) + rms_eps)
        out = x32 @ weight.float().T
        if bias is not None:
            out = out + bias.float()
        if residual is not None:
            residual.copy_((residual.float() + out).to(residual.dtype))
            return residual
        return out.to(out_dtype or x.dtype)

    def rope_kv_write(self, qkv, positions, inv_freq, slots, k_pool, v_pool, num_heads, num_kv_heads,
                      head_dim, write_kv=True):
        tokens = qkv.shape[0]
        page_size = k_pool.shape[2]
        x = qkv.float().view(tokens, num_heads + 2 * num_kv_heads, head_dim)
        angles = positions.float()[:, None] * inv_freq[None, :]
        cos = torch.cat((angles, angles), -1).cos()[:, None, :]
        sin = torch.cat((angles, angles), -1).sin()[:, None, :]
        half = head_dim // 2

        def rotate(t):
            return t * cos + torch.cat((-t[..., half:], t[..., :half]), -1) * sin

        q = rotate(x[:, :num_heads])
        k = rotate(x[:, num_heads:num_heads + num_kv_heads])
        v = x[:, num_heads + num_kv_heads:]
        if write_kv:
            for t in range(tokens):
                slot = int(slots[t])
                if slot < 0:
                    continue
                page, offset = divmod(slot, page_size)
                k_pool[page, :, offset, :] = k[t].to(k_pool.dtype)
                v_pool[page, :, offset, :] = v[t].to(v_pool.dtype)
        return q.reshape(tokens, num_heads * head_dim).to(qkv.dtype)

    def rope_paged_attention(self, qkv, positions, inv_freq, slots, k_pool, v_pool, batch, num_heads, num_kv_heads,
                             head_dim, scale, window=None, write_kv=True):
        q = self.rope_kv_write(qkv, positions, inv_freq, slots, k_pool, v_pool, num_heads, num_kv_heads, head_dim,
                               write_kv)
        return self.paged_attention(q, k_pool, v_pool, batch, num_heads, num_kv_heads, head_dim, scale, window)

    def paged_attention(self, q, k_pool, v_pool, batch, num_heads, num_kv_heads, head_dim, scale, window,
                        value_dim=None):
        page_size = k_pool.shape[2]
        group = num_heads // num_kv_heads
        out = torch.empty((q.shape[0], num_heads * (value_dim or head_dim)), dtype=q.dtype)
        q3 = q.float().view(-1, num_heads, head_dim)
        for seg in range(batch.num_segments):
            start, length, pos0 = (int(batch.seg_q_start[seg]), int(batch.seg_q_len[seg]),
                                   int(batch.seg_pos0[seg]))
            table = batch.block_table[int(batch.seg_slot[seg])]
            for r in range(length):
                p = pos0 + r
                low = max(0, p - window + 1) if window else 0
                keys = torch.arange(low, p + 1)
                pages = table[(keys // page_size).long()].long()
                assert (pages >= 0).all(), "attention reads a page the request does not hold"
                offsets = (keys % page_size).long()
                k = k_pool[pages, :, offsets, :].float()   # [keys, kv_heads, D]
                v = v_pool[pages, :, offsets, :].float()
                k = k.repeat_interleave(group, dim=1)
                v = v.repeat_interleave(group, dim=1)
                scores = torch.einsum("hd,khd->hk", q3[start + r], k) * scale
                probabilities = torch.softmax(scores, dim=-1)
                out[start + r] = torch.einsum("hk,khd->hd", probabilities, v).reshape(-1).to(q.dtype)
        return out

    def sample(self, logits, temperatures, seeds, counters):
        from plain_qwen2 import temperature_sample, uniform_from_seed

        tokens = torch.empty(logits.shape[0], dtype=torch.int32)
        for row in range(logits.shape[0]):
            temperature = float(temperatures[row])
            if temperature <= 0:
                tokens[row] = int(torch.argmax(logits[row]))
            else:
                u = uniform_from_seed(int(seeds[row]) & ((1 << 64) - 1), int(counters[row]))
                tokens[row] = temperature_sample(logits[row], temperature, u)[0]
        return tokens

    # ---- the kernels of 32-bit-stream models with shifts, recurrences and differential attention
    def embedding_positions(self, ids, positions, table, position_table):
        return table[ids.long()].float() + position_table[positions.long()].float()

    def scalar_rms_norm(self, x, gain, eps, out_dtype, want_float=False):
        out = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * gain
        return (out, out.to(out_dtype)) if want_float else out.to(out_dtype)

    def token_shift(self, a, coefficients, state, ctx, out_dtype):
        out = torch.empty((coefficients.shape[0], *a.shape), dtype=torch.float32)
        for segment in ctx.segments:
            rows = slice(segment.row_start, segment.row_start + segment.length)
            previous = torch.cat([state[segment.slot][None], a[rows][:-1]], dim=0)
            out[:, rows] = a[rows][None] + (previous - a[rows])[None] * coefficients[:, None, :]
            state[segment.slot] = a[rows][-1]
        return out.to(out_dtype)

    def bonus_recurrence(self, r, k, v, decay_raw, gate_raw, decay_bias, bonus, weight, eps, state, ctx, heads, dim,
                         out_dtype):
        out = torch.empty((r.shape[0], heads * dim), dtype=torch.float32)
        w = torch.exp(-torch.exp(decay_raw + decay_bias))
        u = bonus.view(heads, dim)
        for segment in ctx.segments:
            S = state[segment.slot]
            for row in range(segment.row_start, segment.row_start + segment.length):
                kv = k[row].view(heads, dim, 1) * v[row].view(heads, 1, dim)
                o = torch.einsum("hi,hij->hj", r[row].view(heads, dim), S + u[:, :, None] * kv)
                S = w[row].view(heads, dim, 1) * S + kv
                o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps)
                out[row] = o.reshape(-1) * weight * torch.nn.functional.silu(gate_raw[row])
            state[segment.slot] = S
        return out.to(out_dtype)

    def forget_gate_recurrence(self, q_raw, forget_raw, v, forget_bias, lower, weight, eps, state, ctx, heads, dim,
                               vdim, out_dtype):
        out = torch.empty((q_raw.shape[0], heads * vdim), dtype=torch.float32)
        f = lower + (1 - lower) * torch.sigmoid(forget_raw + forget_bias)
        q = torch.nn.functional.silu(q_raw)
        for segment in ctx.segments:
            S = state[segment.slot]
            for row in range(segment.row_start, segment.row_start + segment.length):
                S = f[row].view(heads, dim, 1) * S + (1 - f[row]).view(heads, dim, 1) * v[row].view(heads, 1, vdim)
                o = torch.einsum("hi,hij->hj", q[row].view(heads, dim), S)
                out[row] = (o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * weight).reshape(-1)
            state[segment.slot] = S
        return out.to(out_dtype)

    def add_residual(self, residual, a, b=None):
        residual += a if b is None else a + b
        return residual

    def gated_activation(self, gate_up, block, activation):
        inner = gate_up.shape[1] // 2
        blocks = gate_up.float().view(gate_up.shape[0], inner // block, 2, block)
        gate, up = blocks[:, :, 0].reshape(-1, inner), blocks[:, :, 1].reshape(-1, inner)
        act = torch.nn.functional.silu(gate) if activation == "silu" else torch.nn.functional.gelu(gate, approximate="tanh")
        return (act * up).to(gate_up.dtype)

    def linear_gated(self, x, weight, block, activation):
        return self.gated_activation(self.linear(x, weight), block, activation)

    def tanh_(self, x):
        return x.copy_(torch.tanh(x.float()).to(x.dtype))

    def qk_norm_kv_write(self, qkv, q_weight, k_weight, eps, slots, k_pool, v_pool, heads, kv_heads, dim, vdim,
                         write_kv=True):
        rows, page_size = qkv.shape[0], k_pool.shape[2]
        nq, nk = 2 * heads * dim, 2 * kv_heads * dim

        def normed(t, weight):
            t = t.reshape(rows, -1, dim)
            return (t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * weight).reshape(rows, -1)

        q = normed(qkv[:, :nq], q_weight)
        k = normed(qkv[:, nq:nq + nk], k_weight).view(rows, kv_heads, 2 * dim)
        v = qkv[:, nq + nk:].reshape(rows, kv_heads, vdim)
        if write_kv:
            for t in range(rows):
                page, offset = divmod(int(slots[t]), page_size)
                k_pool[page, :, offset, :] = k[t].to(k_pool.dtype)
                v_pool[page, :, offset, :] = v[t].to(v_pool.dtype)
        return q.to(k_pool.dtype)

    def differential_attention(self, q, k_pool, v_pool, batch, heads, kv_heads, dim, vdim, scale, window, keep_first,
                               lam, eps, out_scale):
        page_size, group = k_pool.shape[2], heads // kv_heads
        out = torch.empty((q.shape[0], heads * vdim), dtype=q.dtype)
        q4 = q.float().view(-1, heads, 2, dim)
        for seg in range(batch.num_segments):
            start, length, pos0 = int(batch.seg_q_start[seg]), int(batch.seg_q_len[seg]), int(batch.seg_pos0[seg])
            table = batch.block_table[int(batch.seg_slot[seg])]
            for r in range(length):
                p = pos0 + r
                keys = torch.tensor([j for j in range(p + 1) if not window or p - j < window or j < keep_first])
                pages = table[(keys // page_size).long()].long()
                assert (pages >= 0).all(), "attention reads a page the request does not hold"
                offsets = (keys % page_size).long()
                k = k_pool[pages, :, offsets, :].float().view(len(keys), kv_heads, 2, dim).repeat_interleave(group, dim=1)
                v = v_pool[pages, :, offsets, :].float().repeat_interleave(group, dim=1)
                weights = torch.softmax(torch.einsum("hmd,khmd->hmk", q4[start + r], k) * scale, dim=-1)
                maps = torch.einsum("hmk,khd->hmd", weights, v)
                o = maps[:, 0] - lam * maps[:, 1]
                o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * out_scale
                out[start + r] = o.reshape(-1).to(q.dtype)
        return out

    # ---- 32-bit stream between layer norms, latent attention
    def embedding_rows32(self, ids, table, scale=1.0):
        return table[ids.long()].float() * scale

    @staticmethod
    def _layer_norm(v, pair, eps):
        mean = v.mean(-1, keepdim=True)
        centred = v - mean
        return centred * torch.rsqrt((centred * centred).mean(-1, keepdim=True) + eps) * pair[0] + pair[1]

    def layer_norm_step(self, x, eps, *, delta=None, delta_norm=None, offset=None, norm=None, out_dtype=None):
        if delta is not None:
            x += self._layer_norm(delta, delta_norm, eps)
        if offset is not None:
            x += offset
        return None if norm is None else self._layer_norm(x, norm, eps).to(out_dtype or torch.float32)

    def add_rows(self, x, vector):
        x += vector
        return x

    def clamped_gate(self, gate_up, block, limit, slope):
        inner = gate_up.shape[1] // 2
        blocks = gate_up.float().view(gate_up.shape[0], inner // block, 2, block)
        gate, up = blocks[:, :, 0].reshape(-1, inner), blocks[:, :, 1].reshape(-1, inner)
        gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
        return (gate * torch.sigmoid(slope * gate) * (up + 1.0)).to(gate_up.dtype)

    def linear_clamped_gate(self, x, weight, block, limit, slope):
        return self.clamped_gate(self.linear(x, weight), block, limit, slope)

    def scale_(self, x, factor):
        x *= factor
        return x

    @staticmethod
    def _turn(vector, positions, frequencies, interleaved):
        """vector [rows, ..., n]: the first 2 * len(frequencies) entries turned by the rows' positions."""
        pairs = frequencies.shape[0]
        out = vector.clone()
        angle = positions.float()[:, None] * frequencies[None, :]
        shape = (vector.shape[0],) + (1,) * (vector.dim() - 2) + (pairs,)
        cos, sin = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
        first = torch.arange(pairs) * 2 if interleaved else torch.arange(pairs)
        second = first + 1 if interleaved else first + pairs
        u, v = vector[..., first], vector[..., second]
        out[..., first] = u * cos - v * sin
        out[..., second] = v * cos + u * sin
        return out

    def latent_prepare(self, down, q_at, q_rank, c_at, rank, rot, q_weight, c_weight, eps, positions, frequencies,
                       interleaved, slots, pool, write=True):
        def normed(t, weight):
            return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * weight

        q_latent = normed(down[:, q_at:q_at + q_rank], q_weight).to(pool.dtype)
        if write:
            latent = normed(down[:, c_at:c_at + rank], c_weight)
            turned = self._turn(down[:, c_at + rank:c_at + rank + rot], positions, frequencies, interleaved)
            rows, page_size = torch.cat([latent, turned], dim=1).to(pool.dtype), pool.shape[2]
            for t in range(down.shape[0]):
                page, offset = divmod(int(slots[t]), page_size)
                pool[page, 0, offset, :] = rows[t]
        return q_latent

    def absorb_queries(self, q, weight, heads, dim, rot, rank, positions, frequencies, interleaved):
        q = q.view(-1, heads, dim + rot)
        plain = torch.einsum("rhd,hdc->rhc", q[..., :dim], weight.float().view(heads, dim, rank))
        turned = self._turn(q[..., dim:], positions, frequencies, interleaved)
        return torch.cat([plain, turned], dim=-1).reshape(q.shape[0], -1).to(weight.dtype)

    def latent_values(self, mixed, weight, heads, vdim, rank, gate, gate_per_head):
        out = torch.einsum("rhc,hvc->rhv", mixed.view(-1, heads, rank), weight.float().view(heads, vdim, rank))
        gate = torch.sigmoid(gate.float())
        out = out * (gate[:, :, None] if gate_per_head else gate.view(-1, heads, vdim))
        return out.reshape(mixed.shape[0], -1).to(weight.dtype)

    def latent_attention(self, q, pool, batch, heads, rank, rot, scale, window, sink):
        page_size = pool.shape[2]
        out = torch.empty((q.shape[0], heads * rank), dtype=torch.float32)
        q3 = q.float().view(-1, heads, rank + rot)
        for seg in range(batch.num_segments):
            start, length, pos0 = int(batch.seg_q_start[seg]), int(batch.seg_q_len[seg]), int(batch.seg_pos0[seg])
            table = batch.block_table[int(batch.seg_slot[seg])]
            for r in range(length):
                p = pos0 + r
                keys = torch.arange(max(0, p - window + 1) if window else 0, p + 1)
                pages = table[(keys // page_size).long()].long()
                assert (pages >= 0).all(), "attention reads a page the request does not hold"
                rows = pool[pages, 0, (keys % page_size).long(), :].float()
                scores = torch.einsum("hd,kd->hk", q3[start + r], rows) * scale
                if sink is not None:
                    scores = torch.cat([scores, sink[:, None]], dim=1)
                weights = torch.softmax(scores, dim=-1)[:, :len(keys)]
                out[start + r] = (weights @ rows[:, :rank]).reshape(-1)
        return out

    # ---- attention with normalised, turned values; routed experts
    def rotated_prepare(self, qkv, positions, q_weight, k_weight, eps, key_freq, magnitude, value_freq, interleaved,
                        normalise_values, slots, k_pool, v_pool, heads, kv_heads, dim, vdim, write_kv=True):
        def normed(t, weight):
            return t if weight is None else t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * weight

        def turned(t, frequencies, factor):
            full = self._turn(t, positions, frequencies, interleaved)
            n = 2 * frequencies.shape[0]
            if factor != 1.0:
                full[..., :n] = full[..., :n] * factor
            return full

        rows = qkv.shape[0]
        q = turned(normed(qkv[:, :heads * dim], q_weight).view(rows, heads, dim), key_freq, magnitude)
        k = turned(normed(qkv[:, heads * dim:(heads + kv_heads) * dim], k_weight).view(rows, kv_heads, dim), key_freq,
                   magnitude)
        v = qkv[:, (heads + kv_heads) * dim:].view(rows, kv_heads, vdim)
        if normalise_values:
            v = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)
        if value_freq is not None:
            v = turned(v, value_freq, 1.0)
        if write_kv:
            page_size = k_pool.shape[2]
            for t in range(rows):
                slot = int(slots[t])
                if slot < 0:
                    continue
                page, offset = divmod(slot, page_size)
                k_pool[page, :, offset, :] = k[t].to(k_pool.dtype)
                v_pool[page, :, offset, :] = v[t].to(v_pool.dtype)
        return q.reshape(rows, heads * dim).to(k_pool.dtype)

    def turn_heads(self, x, positions, freq, heads, dim, interleaved, sign=1.0):
        turned = self._turn(x.float().view(-1, heads, dim), positions, freq * sign, interleaved)
        x.copy_(turned.reshape(x.shape).to(x.dtype))
        return x

    def route_experts(self, x, router, correction, top, groups=1, keep=1, scoring="softmax", renormalise=False,
                      group_top=1, renorm_eps=0.0):
        logits = x.float() @ router.T
        scores = torch.softmax(logits, dim=-1) if scoring == "softmax" else torch.sigmoid(logits)
        choice = scores if correction is None else scores + correction
        experts = router.shape[0]
        if keep < groups:
            best = choice.view(-1, groups, experts // groups).topk(min(group_top, experts // groups), dim=-1).values.sum(-1)
            kept = torch.zeros_like(best, dtype=torch.bool).scatter_(1, best.topk(keep, dim=-1).indices, True)
            choice = choice.masked_fill(~kept.repeat_interleave(experts // groups, dim=1), float("-inf"))
        chosen = choice.topk(top, dim=-1).indices
        weights = scores.gather(1, chosen)
        if renormalise:
            weights = weights / (weights.sum(-1, keepdim=True) + renorm_eps)
        return chosen.to(torch.int32), weights

    def routed_experts(self, x, chosen, weights, gate_up, down, block, activation="silu"):
        out = torch.zeros((x.shape[0], down.shape[1]), dtype=torch.float32)
        for row in range(x.shape[0]):
            for t in range(chosen.shape[1]):
                e = int(chosen[row, t])
                hidden = self.gated_activation(self.linear(x[row:row + 1], gate_up[e]), block, activation)
                out[row] += weights[row, t] * (hidden.float() @ down[e].float().T)[0]
        return out

    # ---- 32-bit stream with RMS norms behind the sublayers
    @staticmethod
    def _rms(v, eps):
        return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)

    def rms_norm_step(self, x, eps, *, delta=None, delta_weight=None, norm_weight=None, out_dtype=None):
        if delta is not None:
            x += self._rms(delta, eps) * delta_weight
        if out_dtype is None:
            return None
        return (x.clone() if norm_weight is None else self._rms(x, eps) * norm_weight).to(out_dtype)

    def normed_mean(self, a, a_weight, b, b_weight, eps, factor):
        return factor * (self._rms(a, eps) * a_weight + self._rms(b, eps) * b_weight)

    # ---- plain-headed attention: prepare; sigmoid weights
    def head_norm_kv_write(self, qkv, q_weight, k_weight, eps, slots, k_pool, v_pool, heads, kv_heads, dim, vdim,
                           write_kv=True, *, other_values=None, mix=None):
        rows, page_size = qkv.shape[0], k_pool.shape[2]
        nq, nk = heads * dim, kv_heads * dim
        q = self._rms(qkv[:, :nq].reshape(rows, heads, dim), eps)
        k = self._rms(qkv[:, nq:nq + nk].reshape(rows, kv_heads, dim), eps)
        if q_weight is not None:
            q = q * q_weight
        if k_weight is not None:
            k = k * k_weight
        v = qkv[:, nq + nk:]
        if other_values is not None:
            v = (1.0 - mix[0]) * v + mix[0] * other_values
        v = v.reshape(rows, kv_heads, vdim)
        if write_kv:
            for t in range(rows):
                slot = int(slots[t])
                if slot < 0:
                    continue
                page, offset = divmod(slot, page_size)
                k_pool[page, :, offset, :] = k[t].to(k_pool.dtype)
                v_pool[page, :, offset, :] = v[t].to(v_pool.dtype)
        return q.reshape(rows, nq).to(k_pool.dtype)

    def sigmoid_attention(self, q, k_pool, v_pool, batch, heads, kv_heads, dim, vdim, scale, *, distance=None,
                          score_bias=None, head_mix=None):
        page_size = k_pool.shape[2]
        group = heads // kv_heads
        out = torch.empty((q.shape[0], heads * vdim), dtype=q.dtype)
        q3 = q.float().view(-1, heads, dim)
        for seg in range(batch.num_segments):
            start, length, pos0 = int(batch.seg_q_start[seg]), int(batch.seg_q_len[seg]), int(batch.seg_pos0[seg])
            table = batch.block_table[int(batch.seg_slot[seg])]
            for r in range(length):
                p = pos0 + r
                keys = torch.arange(0, p + 1)
                pages = table[(keys // page_size).long()].long()
                assert (pages >= 0).all(), "attention reads a page the request does not hold"
                offsets = (keys % page_size).long()
                k = k_pool[pages, :, offsets, :].float().repeat_interleave(group, dim=1)
                v = v_pool[pages, :, offsets, :].float().repeat_interleave(group, dim=1)
                scores = torch.einsum("hd,khd->hk", q3[start + r], k) * scale
                if distance is not None:
                    r1, r2 = distance
                    scores = scores - r1[:, None] * torch.log1p(r2[:, None] * (p - keys).float()[None, :])
                if score_bias is not None:
                    scores = scores + score_bias[:, None]
                weights = torch.sigmoid(scores)
                if head_mix is not None:
                    weights = head_mix @ weights
                out[start + r] = torch.einsum("hk,khd->hd", weights, v).reshape(-1).to(q.dtype)
        return out

    # ---- state-space mixer
    def causal_conv(self, u, weight, bias, state, ctx, activation="silu"):
        taps = weight.shape[1]
        out = torch.empty(u.shape, dtype=torch.float32)
        for segment in ctx.segments:
            rows = slice(segment.row_start, segment.row_start + segment.length)
            padded = torch.cat([state[segment.slot], u[rows]], dim=0)
            total = torch.zeros((segment.length, u.shape[1]), dtype=torch.float32)
            if bias is not None:
                total = total + bias
            for tap in range(taps):
                total = total + padded[tap:tap + segment.length] * weight[:, tap]
            out[rows] = torch.nn.functional.silu(total) if activation == "silu" else total
            state[segment.slot] = padded[-(taps - 1):]
        return out

    def state_space_scan(self, x, B, C, dt_raw, dt_bias, A_log, D, state, ctx, heads, vdim, n, groups):
        y = torch.empty((x.shape[0], heads * vdim), dtype=torch.float32)
        dt = torch.nn.functional.softplus(dt_raw + dt_bias)
        decay = torch.exp(-torch.exp(A_log) * dt)
        per = heads // groups
        for segment in ctx.segments:
            S = state[segment.slot]                   # [heads, vdim, n]
            for row in range(segment.row_start, segment.row_start + segment.length):
                xr = x[row].view(heads, vdim)
                Br = B[row].view(groups, n).repeat_interleave(per, dim=0)
                Cr = C[row].view(groups, n).repeat_interleave(per, dim=0)
                S = decay[row].view(heads, 1, 1) * S + dt[row].view(heads, 1, 1) * xr[:, :, None] * Br[:, None, :]
                y[row] = (torch.einsum("hpn,hn->hp", S, Cr) + D[:, None] * xr).reshape(-1)
            state[segment.slot] = S
        return y

    def gated_group_norm(self, y, gate, weight, eps, parts, out_dtype):
        v = y if gate is None else y * torch.nn.functional.silu(gate)
        rows, inner = v.shape
        v = self._rms(v.reshape(rows, parts, inner // parts), eps).reshape(rows, inner)
        return (v * weight).to(out_dtype)
