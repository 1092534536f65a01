"""Helpers of the Ratilorn tests: small configurations of the tests' own, random weights drawn here
(large enough that attention and routing are peaked and the state-space layers remember), an engine
around the framework's model, cache manager and step function on any device, and the plain oracle
beside it."""

from __future__ import annotations

import math

import torch

import plain_ratilorn as plain
from mini_llm_runtime_b200.cache import CacheManager
from mini_llm_runtime_b200.config import config_from_dict
from mini_llm_runtime_b200.engine import ModelRunner, StepEntry
from mini_llm_runtime_b200.models import build_model

CLOSE_CALL = 0.05      # a router's margin below which a bfloat16 rounding of its input may move the choice
CLOSE_CALL_32 = 1e-4   # the same for a 32-bit engine against the 64-bit oracle


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def heads(count, kv_heads, dim, vdim, scale=None):
    return {"heads": count, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}


def attention(count, kv_heads, dim, vdim, *, scale=None, v_mix=False, mlp=None):
    mixer = heads(count, kv_heads, dim, vdim, scale)
    if v_mix:
        mixer["v_mix"] = True
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def parallel(left, right, mlp=None):
    """right: (heads, vdim, state, groups, conv, norm_groups)."""
    names = ("heads", "vdim", "state", "groups", "conv", "norm_groups")
    return {"type": "parallel", "mixer": {"left": left, "right": dict(zip(names, right))}, "mlp": mlp}


def config(layers, width, vocab, *, eps=1e-5, logit_scale=1.0, max_positions=512):
    return {"architecture": "Ratilorn", "vocab": vocab, "width": width, "max_positions": max_positions,
            "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": list(layers)}


# every size differs from every other; one layer has no feed-forward; dense, grouped and ungrouped routed
# feed-forwards with and without a shared expert; a value blend across layers of different key sizes;
# an attention layer without the blend between the two that have it
MIXED = config([parallel(heads(4, 2, 16, 24), (3, 8, 20, 1, 4, 1), dense(40)),
                attention(6, 2, 12, 8, scale=0.3, v_mix=True, mlp=moe(24, 6, 2, groups=(3, 2), shared=16)),
                attention(3, 3, 8, 12),
                parallel(heads(2, 1, 24, 16, 0.25), (4, 6, 18, 2, 2, 2), moe(32, 8, 3, groups=(4, 2))),
                attention(6, 2, 10, 8, v_mix=True, mlp=moe(20, 4, 2, shared=8))],
               width=96, vocab=131, logit_scale=1.5)
# sizes that are no multiple of 8, one head, a single chosen expert, a state smaller than a thread's share
ODD = config([parallel(heads(1, 1, 10, 6), (1, 5, 7, 1, 3, 1), moe(52, 5, 1, shared=12)),
              attention(3, 1, 6, 14, v_mix=True, mlp=dense(20)),
              attention(3, 1, 6, 14, scale=0.5, v_mix=True)],
             width=68, vocab=77, eps=3e-6, logit_scale=0.7)
# equal sizes everywhere (values a given model may happen to make equal), one group that is kept, no blend,
# every expert chosen (no choice hangs on a rounding: one expert of two would be the whole feed-forward)
PLAIN = config([parallel(heads(2, 2, 16, 16), (2, 16, 16, 2, 2, 2), moe(16, 2, 2, groups=(1, 1))),
                attention(2, 2, 16, 16, mlp=moe(16, 2, 2))],
               width=32, vocab=40)
# sizes the tensor-core kernels take (heads of 64 and 128, multiples of 64), for bfloat16 and many rows
WIDE = config([parallel(heads(4, 2, 64, 64), (4, 64, 64, 1, 4, 2), moe(128, 8, 2, groups=(4, 2), shared=128)),
               attention(4, 2, 128, 64, v_mix=True, mlp=dense(256)),
               parallel(heads(2, 1, 128, 128), (8, 32, 128, 2, 4, 1), moe(192, 4, 3)),
               attention(8, 2, 64, 64, v_mix=True)],
              width=256, vocab=520, eps=1e-6, logit_scale=2.0)


def draw_tensors(expected, seed, overrides=None):
    """Random weights by name and by the kind each part declares, stored as bfloat16 (so that the 32-bit
    and the 16-bit engine and the oracle all read the same numbers).  Routers are strong so that a
    rounding of their input rarely moves a choice; decays are slow enough that a lost state shows."""
    generator = torch.Generator().manual_seed(seed)

    def normal(shape, scale=1.0):
        return torch.randn(shape, generator=generator) * scale

    def uniform(shape, low, high):
        return low + (high - low) * torch.rand(shape, generator=generator)

    tensors = {}
    for name in sorted(expected):
        spec = expected[name]
        shape = tuple(spec.shape)
        last = name.rsplit(".", 1)[-1]
        if last in ("r1", "r2"):
            value = uniform(shape, 0.2, 1.2)
        elif last == "pb":
            value = normal(shape, 0.5) - 1.0
        elif last == "talk":
            value = torch.eye(shape[0]) + normal(shape, 0.3)
        elif last == "vmix":
            value = uniform(shape, 0.25, 0.75)
        elif last == "A_log":
            value = uniform(shape, -3.0, 0.5)
        elif last == "dt_bias":
            value = normal(shape, 0.5)
        elif last == "conv":
            value = normal(shape, 0.6)
        elif last == "correction":
            value = normal(shape, 0.3)          # wide apart, so that few choices hang on a rounding where the scores saturate
        elif last == "router":
            value = normal(shape, 3.0 / math.sqrt(shape[-1]))
        elif name.endswith((".norm1", ".norm2", "final.norm")):
            value = normal(shape, 0.3)                    # stored as an offset from one
        elif spec.init == "norm":
            value = 1.0 + normal(shape, 0.2)
        elif spec.init == "bias":
            value = normal(shape, 0.5)
        else:
            fan_in = shape[-1] if len(shape) > 1 else 1
            value = normal(shape, 1.2 / math.sqrt(fan_in))
        tensors[name] = value
    for name in ("embed", "pos"):
        if name in tensors:
            tensors[name] = normal(tensors[name].shape, 1.0 if name == "embed" else 0.5)
    for name, value in (overrides or {}).items():
        tensors[name] = value(tensors[name]) if callable(value) else value
    return {name: value.to(torch.bfloat16) for name, value in tensors.items()}


def tokens_for(vocab, length, seed):
    return torch.randint(0, vocab, (length,), generator=torch.Generator().manual_seed(seed)).tolist()


def row_errors(got, want):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    delta = got - want
    delta = delta - delta.mean(dim=-1, keepdim=True)
    return delta.pow(2).mean(dim=-1).sqrt() / float(want.std())


class Logits(torch.Tensor):
    """The oracle's logits with, per row, the smallest margin of any router's choice."""

    margin = None


def take(want, index):
    out = torch.Tensor.__getitem__(want, index).as_subclass(Logits)
    out.margin = None if want.margin is None else want.margin[index]
    return out


def assert_logits_close(got, want, dtype, what="", limit=None):
    """Difference of the rows with their mean taken off, root mean square over the vocabulary, relative to
    the logits' own spread: 2e-5 in 32-bit (order of additions only), 4e-2 in bfloat16 (the test models are
    narrow: a rounding weighs more than in a wide one).  A router's close
    call may go the other way in the engine (its input is rounded; in 32-bit a gap of a millionth is
    enough): such rows are left out, and the rows behind them (which read them through the attention and
    the carried state) get ten times the allowance in bfloat16, which still tells a wrong kernel from a
    rounding, and are left out in 32-bit, where a changed choice is no rounding any more."""
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} against {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    error = row_errors(got, want)
    limit = limit or (2e-5 if dtype == torch.float32 else 4e-2)
    margin = getattr(want, "margin", None)
    close = CLOSE_CALL_32 if dtype == torch.float32 else CLOSE_CALL
    if margin is not None and bool((margin < close).any()):
        settled = margin >= close
        later = torch.cumsum((~settled).long(), dim=0) > 0
        if dtype == torch.float32:
            assert not bool(later[:len(later) // 2].any()), f"{what}: a router's tie in the first half; use another seed"
            error = torch.where(later, torch.zeros_like(error), error)
        else:
            error = torch.where(settled, torch.where(later, error / 10.0, error), torch.zeros_like(error))
    worst = int(error.argmax())
    assert float(error.max()) <= limit, f"{what}: row {worst} is off by {float(error.max()):.3e} (allowed {limit:.0e})"


def plain_logits(config_dict, tensors, tokens):
    """The oracle's logits with the routers' margins per row."""
    margins = []
    original = plain.route

    def recording(h, t, prefix, router):
        chosen, weights, _ = original(h, t, prefix, router)
        rows = [original(h[i:i + 1], t, prefix, router)[2] for i in range(h.shape[0])]
        margins.append(torch.tensor(rows, dtype=torch.float64))
        return chosen, weights, min(rows)

    plain.route = recording
    try:
        logits, _ = plain.forward(config_dict, tensors, tokens)
    finally:
        plain.route = original
    logits = logits.as_subclass(Logits)
    logits.margin = (torch.stack(margins).min(dim=0).values if margins
                     else torch.full((len(tokens),), math.inf, dtype=torch.float64))
    return logits


class REngine:
    def __init__(self, config_dict, dtype, device, *, page_size=16, num_pages=64, max_requests=4, max_tokens=512,
                 seed=0, overrides=None, max_step_tokens=None):
        self.config_dict = config_dict
        self.dtype = dtype
        self.device = device
        self.config = config_from_dict(config_dict)
        self.model = build_model(self.config, dtype)
        self.tensors = draw_tensors(self.model.expected_tensors(), seed, overrides)
        self.model.load(self.tensors, device)
        self.cache = CacheManager(self.model.cache_needs(), page_size=page_size, num_pages=num_pages,
                                  max_requests=max_requests, max_tokens_per_request=max_tokens, dtype=dtype,
                                  device=device, max_step_tokens=max_step_tokens or max_tokens)
        self.runner = ModelRunner(self.model, self.cache)
        self.runner.graph_capture_after = 1

    def plain(self, tokens, config_dict=None, tensors=None):
        return plain_logits(config_dict or self.config_dict, tensors or self.tensors, tokens)

    def step(self, entries):
        """entries: (request id, tokens, wanted places)."""
        return self.runner.step([StepEntry(rid, list(toks), list(want)) for rid, toks, want in entries])

    def run_cuts(self, request_id, tokens, cuts, release=True):
        self.cache.create_request(request_id)
        outputs, start = [], 0
        for end in list(cuts) + [len(tokens)]:
            if end <= start:
                continue
            outputs.append(self.step([(request_id, tokens[start:end], range(end - start))]))
            start = end
        if release:
            self.cache.release(request_id)
        return torch.cat(outputs)

    def run_plan(self, prompts, plan):
        """Several requests side by side: ``plan`` is a list of {name: tokens this step}; returns the
        logits of every request's tokens in order."""
        got = {name: [] for name in prompts}
        at = {name: 0 for name in prompts}
        for step in plan:
            for name in step:
                if at[name] == 0:
                    self.cache.create_request(name)
            entries = [(name, prompts[name][at[name]:at[name] + count], range(count)) for name, count in step.items()]
            logits = self.step(entries)
            row = 0
            for name, count in step.items():
                got[name].append(logits[row:row + count])
                row += count
                at[name] += count
                if at[name] == len(prompts[name]):
                    self.cache.release(name)
        return {name: torch.cat(rows) for name, rows in got.items()}


def dominant_key_case(length, query, key, seed, dim=12, vdim=10, kv_heads=1):
    """A one-layer model (sigmoid attention, no feed-forward) whose weights let one chosen key carry
    nearly all the weight of one chosen query.  Token ids are the positions' own (vocabulary = length),
    position vectors are zero.  Keys are the first ``dim`` channels of the embedding, queries (both heads)
    the same channels rolled by one; the key's token embeds as the query's with those channels rolled,
    so that after the per-head norms q_query . k_key = dim while any other pair scores about sqrt(dim)
    at most.  With a score scale of 24 / dim (2 at the default size), a score bias 10 below the matched
    score and no distance bias, that key gets a weight near 1 and every other key (the query's own
    included) a small one: the query's output is that key's value, whenever the key is seen, however far
    back it lies."""
    width = max(40, dim + 8)
    scale = 24.0 / dim if dim <= 12 else 32.0 / dim
    bias = -(scale * dim - 10.0)
    cfg = config([attention(2 * kv_heads, kv_heads, dim, vdim, scale=scale)], width=width, vocab=length, max_positions=length)
    generator = torch.Generator().manual_seed(seed)

    def embed(table):
        table = torch.randn(table.shape, generator=generator)
        table[key, :dim] = torch.roll(table[query, :dim], 1)
        return table

    def key_matrix(_):
        return torch.cat([torch.eye(dim), torch.zeros(dim, width - dim)], dim=1)

    def query_matrix(_):
        rolled = torch.cat([torch.roll(torch.eye(dim), 1, dims=0), torch.zeros(dim, width - dim)], dim=1)
        return torch.cat([rolled] * (2 * kv_heads))

    def key_matrices(_):
        return torch.cat([key_matrix(_)] * kv_heads)

    zero = torch.zeros_like
    overrides = {"embed": embed, "pos": zero, "l0.norm1": zero, "l0.mix.k": key_matrices, "l0.mix.q": query_matrix,
                 "l0.mix.q.b": zero, "l0.mix.k.b": zero, "l0.mix.r1": zero, "l0.mix.pb": lambda t: torch.full_like(t, bias),
                 "l0.mix.talk": lambda t: torch.eye(t.shape[0])}
    return cfg, overrides


def random_config(seed):
    """A configuration drawn from a seed: sizes of every parity, both layer kinds in any order, layers
    with and without a feed-forward, dense and routed ones, value blends."""
    import random

    rng = random.Random(seed)
    layers = []
    blend = (rng.randint(1, 2), rng.choice([4, 6, 12]))      # kv heads and value size of the layers that blend
    for _ in range(rng.randint(1, 4)):
        kind = rng.choice(["dense", "moe", "moe", None])
        mlp = None
        if kind == "dense":
            mlp = dense(rng.choice([8, 20, 36]))
        elif kind == "moe":
            groups = rng.choice([None, (1, 1), (2, 1), (2, 2), (3, 2)])
            per_group = rng.randint(1, 3)
            experts = per_group * (groups[0] if groups else rng.randint(1, 3))
            eligible = per_group * groups[1] if groups else experts
            mlp = moe(rng.choice([8, 20, 24]), experts, rng.randint(1, eligible), groups, rng.choice([None, 8, 12]))
        if rng.random() < 0.5:
            if rng.random() < 0.6:
                kv_heads, vdim = blend
                layers.append(attention(kv_heads * rng.randint(1, 3), kv_heads, rng.choice([4, 6, 10, 16]), vdim,
                                        scale=rng.choice([None, 0.3]), v_mix=True, mlp=mlp))
            else:
                kv_heads = rng.randint(1, 3)
                layers.append(attention(kv_heads * rng.randint(1, 2), kv_heads, rng.choice([4, 8, 10]),
                                        rng.choice([2, 6, 8, 20]), mlp=mlp))
        else:
            kv_heads = rng.randint(1, 2)
            groups = rng.randint(1, 2)
            state_heads = groups * rng.randint(1, 2)
            vdim = rng.choice([4, 6, 10])
            norm_groups = rng.choice([g for g in (1, 2, state_heads) if (state_heads * vdim) % g == 0])
            layers.append(parallel(heads(kv_heads * rng.randint(1, 3), kv_heads, rng.choice([4, 8, 16]), rng.choice([4, 6, 12]),
                                         rng.choice([None, 0.4])),
                                   (state_heads, vdim, rng.choice([3, 8, 17, 40]), groups, rng.randint(2, 5), norm_groups), mlp))
    return config(layers, width=rng.choice([24, 36, 64, 72]), vocab=rng.choice([31, 64, 100]),
                  eps=rng.choice([1e-6, 1e-5, 1e-3]), logit_scale=rng.choice([0.5, 1.0, 3.0]))
