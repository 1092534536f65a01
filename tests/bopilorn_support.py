"""Helpers of the Bopilorn tests: small configurations of the tests' own, random weights drawn here
(large enough that attention and routing are peaked), an engine around the framework's model, cache
manager and step function on any device, and the plain oracle beside it."""

from __future__ import annotations

import math

import torch

import plain_bopilorn as plain
from mini_llm_runtime_b200.cache import CacheManager
from mini_llm_runtime_b200.config import config_from_dict
from mini_llm_runtime_b200.engine import ModelRunner, StepEntry
from mini_llm_runtime_b200.models import build_model


def moe(ff, experts, top, groups=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def attention(heads, kv_heads, dim, vdim, *, base=10000.0, scale=None, dims=None, scaling=None, mlp=None):
    rot = {"base": base, "dims": dim if dims is None else dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                      "scale": scale if scale is not None else 1.0 / math.sqrt(dim), "rot": rot},
            "mlp": mlp}


def config(layers, width, vocab, *, eps=1e-5, embedding_scale=1.0):
    return {"architecture": "Bopilorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embedding_scale}, "layers": list(layers)}


# every size differs from every other; one layer has no feed-forward; grouped and ungrouped routers;
# scaled and plain frequencies; a rotation over a part of the head
MIXED = config([attention(4, 2, 16, 24, scaling=(4.0, 64.0, 8.0, 1.0), mlp=moe(40, 6, 2, groups=(3, 2))),
                attention(3, 3, 8, 12, base=500.0, dims=6, scale=0.4, mlp=moe(24, 4, 3)),
                attention(6, 2, 12, 8, dims=4, scaling=(2.5, 30.0, 4.0, 0.5)),
                attention(2, 1, 24, 16, base=77.0, mlp=moe(32, 8, 2, groups=(4, 1)))],
               width=96, vocab=131, embedding_scale=2.5)
# sizes that are no multiple of 8, one head, a single chosen expert, experts that do not fill a warp
ODD = config([attention(1, 1, 10, 6, dims=6, mlp=moe(52, 5, 1)), attention(3, 1, 6, 14, base=90.0, mlp=moe(20, 3, 3))],
             width=68, vocab=77, eps=3e-6, embedding_scale=0.7)
# equal sizes everywhere (values a given model may happen to make equal), one group that is kept
PLAIN = config([attention(2, 2, 16, 16, mlp=moe(16, 2, 1, groups=(1, 1))), attention(2, 2, 16, 16, mlp=moe(16, 2, 2))],
               width=32, vocab=40)
# sizes the tensor-core kernels take (heads of 64 and 128, multiples of 64), for bfloat16 and many rows
WIDE = config([attention(4, 2, 64, 64, scaling=(2.0, 256.0, 16.0, 1.0), mlp=moe(128, 8, 2, groups=(4, 2))),
               attention(2, 1, 128, 128, base=2000.0, dims=64, mlp=moe(192, 4, 3)),
               attention(4, 4, 64, 128, base=300.0)],
              width=256, vocab=520, eps=1e-6, embedding_scale=1.5)


def draw_tensors(expected, seed, overrides=None):
    """Random weights by the kind each part declares, stored as bfloat16 (so that the 32-bit and the
    16-bit engine and the oracle all read the same numbers).  Routers are strong (logits several
    units apart) so that a rounding of their input does not move a choice; corrections are small
    but of either sign."""
    generator = torch.Generator().manual_seed(seed)
    tensors = {}
    for name in sorted(expected):
        spec = expected[name]
        shape = tuple(spec.shape)
        if spec.init == "norm":
            value = 1.0 + 0.2 * torch.randn(shape, generator=generator)
        elif name.endswith(".correction"):
            value = 0.05 * torch.randn(shape, generator=generator)
        elif spec.init == "bias":
            value = 0.5 * torch.randn(shape, generator=generator)
        elif name.endswith(".router"):
            value = torch.randn(shape, generator=generator) * (3.0 / math.sqrt(shape[-1]))
        else:
            fan_in = shape[-1] if len(shape) > 1 else 1
            value = torch.randn(shape, generator=generator) * (1.2 / math.sqrt(fan_in))
        tensors[name] = value
    if "embed" in tensors:
        tensors["embed"] = torch.randn(tensors["embed"].shape, generator=generator)
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
    """The oracle's logits with, per row, the weight that hangs on a close call of a router."""

    risk = None


def take(want, index):
    """Rows of the oracle's logits together with their risks."""
    out = torch.Tensor.__getitem__(want, index).as_subclass(Logits)
    out.risk = None if want.risk is None else want.risk[index]
    return out


def assert_logits_close(got, want, dtype, what="", limit=None):
    """Difference of the rows with their mean taken off, root mean square over the vocabulary,
    relative to the logits' own spread: 2e-5 in 32-bit (order of additions only), 3e-2 in bfloat16.
    In bfloat16 a router's close call may go the other way (its input is rounded); rows where an
    expert of some weight hangs on one are left out."""
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} against {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    error = row_errors(got, want)
    limit = limit or (2e-5 if dtype == torch.float32 else 3e-2)
    risk = getattr(want, "risk", None)
    if dtype != torch.float32 and risk is not None and bool((risk > plain.CLOSE_CALL).any()):
        settled = risk <= plain.CLOSE_CALL
        assert float(settled.double().mean()) >= 0.5, f"{what}: too many rows hang on a router's close call"
        # a row whose choice went the other way is another row for all that read it later: those get
        # three times the allowance (measured: 0.05 where the row itself was off by 0.9)
        later = torch.cumsum((~settled).long(), dim=0) > 0
        error = torch.where(settled, torch.where(later, error / 3.0, error), torch.zeros_like(error))
    worst = int(error.argmax())
    assert float(error.max()) <= limit, f"{what}: row {worst} is off by {float(error.max()):.3e} (allowed {limit:.0e})"


class BEngine:
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
        risks = []
        logits = plain.forward(config_dict or self.config_dict, tensors or self.tensors, tokens, risk_out=risks)
        logits = logits.as_subclass(Logits)
        logits.risk = torch.stack(risks).max(dim=0).values if risks else torch.zeros(len(tokens), dtype=torch.float64)
        return logits

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


def dominant_key_case(length, query, key, seed, dim=12, vdim=10):
    """A one-layer model without a feed-forward whose weights let one chosen key dominate one chosen
    query.  Token ids are the positions' own (vocabulary = length).  Only the first two entries of a
    head are turned, and the projections leave them zero, so the scores do not depend on the
    distance.  The key projection is the identity on the input's first dim - 2 channels and the query
    projection of both heads a roll of them by one, under a large score scale; the key's token embeds as the query's with
    those channels rolled, hence k_key ~ roll(k_query): that one key collects nearly all the weight of
    that one query whenever it is visible, and no other key (the query's own included) does.  Values
    are turned by their positions as ever, so a wrong angle on the way back shows too."""
    width = 40
    cfg = config([attention(2, 1, dim, vdim, dims=2, scale=9.0)], width=width, vocab=length)
    generator = torch.Generator().manual_seed(seed)
    inner = dim - 2

    def embed(table):
        table = torch.randn(table.shape, generator=generator)
        table[key, :inner] = torch.roll(table[query, :inner], 1)
        table[key, inner:] = table[query, inner:]
        return table

    def key_matrix(_):
        return torch.cat([torch.zeros(2, width), torch.cat([torch.eye(inner), torch.zeros(inner, width - inner)], dim=1)])

    def query_matrix(_):
        rolled = torch.cat([torch.roll(torch.eye(inner), 1, dims=0), torch.zeros(inner, width - inner)], dim=1)
        per_head = torch.cat([torch.zeros(2, width), rolled])
        return torch.cat([per_head, per_head])

    overrides = {"embed": embed, "l0.norm1": lambda t: torch.ones_like(t), "l0.mix.k": key_matrix, "l0.mix.q": query_matrix,
                 "l0.mix.q.norm": lambda t: torch.ones_like(t), "l0.mix.k.norm": lambda t: torch.ones_like(t)}
    return cfg, overrides


def random_config(seed):
    """A configuration drawn from a seed: sizes of every parity, layers with and without a
    feed-forward, grouped and ungrouped routers, scaled and plain frequencies."""
    import random

    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(1, 4)):
        kv_heads = rng.randint(1, 3)
        heads = kv_heads * rng.randint(1, 3)
        dim, vdim = rng.choice([4, 6, 8, 10, 16, 24]), rng.choice([2, 6, 8, 12, 20])
        mlp = None
        if rng.random() < 0.8:
            groups = rng.choice([None, (1, 1), (2, 1), (2, 2), (3, 2)])
            per_group = rng.randint(1, 3)
            experts = per_group * (groups[0] if groups else rng.randint(1, 3))
            eligible = per_group * groups[1] if groups else experts
            mlp = moe(rng.choice([8, 20, 24, 36]), experts, rng.randint(1, eligible), groups)
        scaling = rng.choice([None, (2.0, 40.0, 8.0, 1.0), (8.0, 16.0, 2.0, 0.25)])
        layers.append(attention(heads, kv_heads, dim, vdim, base=rng.choice([30.0, 1000.0, 50000.0]),
                                scale=rng.choice([None, 0.2, 0.4]), dims=rng.choice([None, dim, max(2, dim - 2)]),
                                scaling=scaling, mlp=mlp))
    return config(layers, width=rng.choice([24, 36, 64, 72]), vocab=rng.choice([31, 64, 100]),
                  eps=rng.choice([1e-6, 1e-5, 1e-3]), embedding_scale=rng.choice([0.5, 1.0, 3.5]))
