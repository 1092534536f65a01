"""Ratilorn through the framework's model, cache manager, step function and kernels, against the
plain implementation (``plain_ratilorn``): each mechanism alone, whole prompts, token-by-token
decoding, portions, mixed batches, reused pages and slots, far keys and page borders with a key made
to dominate, the first tokens, long decoding through captured steps, odd and larger sizes, and greedy
generation through the scheduler and the command line."""

from __future__ import annotations

import json
import math
from types import SimpleNamespace

import pytest
import torch

import plain_ratilorn as plain
import ratilorn_support as rs
from mini_llm_runtime_b200 import ops
from mini_llm_runtime_b200.engine import ContinuousBatchEngine

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
F32 = torch.float32
F64 = torch.float64
BF16 = torch.bfloat16
DTYPES = [torch.float32, torch.bfloat16]


def run_alone(layer, dtype, seed=11, length=61, **options):
    config = rs.config([layer], width=72, vocab=90, logit_scale=1.7, **options)
    engine = rs.REngine(config, dtype, DEVICE, seed=seed)
    tokens = rs.tokens_for(90, length, 5)
    want = engine.plain(tokens)
    rs.assert_logits_close(engine.run_cuts("a", tokens, []), want, dtype, "whole")
    rs.assert_logits_close(engine.run_cuts("b", tokens, [30] + list(range(31, length))), want, dtype, "decoded")
    rs.assert_logits_close(engine.run_cuts("c", tokens, [2, 17, 19, 40]), want, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(6, 2, 16, 24), (3, 3, 10, 6), (1, 1, 8, 8), (8, 1, 12, 20), (4, 4, 40, 36)])
def test_sigmoid_attention_alone(sizes, dtype):
    run_alone(rs.attention(*sizes, scale=0.35), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("left,right", [
    (rs.heads(4, 2, 16, 24), (3, 8, 20, 1, 4, 1)),       # a state that leaves a thread's share partly empty
    (rs.heads(2, 2, 8, 8), (4, 6, 16, 2, 2, 4)),         # two groups, a norm in four parts, two taps
    (rs.heads(3, 1, 12, 4), (2, 40, 7, 1, 5, 1)),        # more value channels than a block takes at once, a tiny state
    (rs.heads(2, 1, 64, 64), (2, 10, 70, 2, 3, 2)),      # a state cut over eight threads; the tensor-core attention's sizes
])
def test_the_parallel_mixer_alone(left, right, dtype):
    run_alone(rs.parallel(left, right), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mlp", [rs.dense(56), rs.moe(56, 6, 2, shared=24), rs.moe(56, 6, 3, groups=(3, 2)),
                                 rs.moe(40, 8, 2, groups=(4, 1), shared=8), rs.moe(64, 3, 1), rs.moe(24, 2, 2, groups=(1, 1))])
def test_the_feed_forward(mlp, dtype):
    tokens = rs.tokens_for(90, 40, 3)
    config = rs.config([rs.attention(2, 1, 8, 8, mlp=mlp)], width=72, vocab=90)
    engine = rs.REngine(config, dtype, DEVICE, seed=2)
    rs.assert_logits_close(engine.run_cuts("a", tokens, [25, 26]), engine.plain(tokens), dtype)


def test_router_kernel_against_its_formula():
    """Groups ranked by the sum of their two best choice scores (one, where a group has one expert),
    negative choice scores, ties, renormalised weights."""
    k = ops.current()
    generator = torch.Generator().manual_seed(3)
    for rows, width, experts, top, groups, keep, group_top in [(7, 40, 8, 3, 4, 2, 2), (150, 64, 12, 4, 3, 2, 2), (5, 24, 6, 2, 6, 3, 2),
                                                              (9, 32, 9, 3, 3, 1, 3), (4, 16, 4, 2, 1, 1, 2)]:
        x = torch.randn(rows, width, generator=generator)
        router = torch.randn(experts, width, generator=generator) * (2.0 / math.sqrt(width))
        correction = torch.randn(experts, generator=generator) * 0.5 - 0.8
        chosen, weights = k.route_experts(x.to(DEVICE), router.to(DEVICE), correction.to(DEVICE), top, groups, keep, "sigmoid",
                                          True, group_top=group_top, renorm_eps=1e-20)
        s = torch.sigmoid(x.double() @ router.double().T)
        c = s + correction.double()
        size = experts // groups
        score = c.view(rows, groups, size).topk(min(group_top, size), dim=-1).values.sum(-1)
        kept = torch.zeros(rows, groups, dtype=torch.bool).scatter_(1, score.topk(keep, dim=-1).indices, True)
        c = c.masked_fill(~kept.repeat_interleave(size, dim=1), -math.inf)
        want = c.topk(top, dim=-1).indices
        assert chosen.cpu().tolist() == want.tolist()
        picked = s.gather(1, want)
        assert torch.allclose(weights.cpu().double(), picked / picked.sum(-1, keepdim=True), atol=1e-6)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 64, 64), (16, 4, 128, 128), (14, 2, 64, 128), (3, 1, 128, 64),
                                                     (6, 2, 24, 40), (5, 5, 10, 6)])
def test_sigmoid_attention_kernels_against_their_formula(heads, kv_heads, dim, vdim):
    """The float32 kernel, the bfloat16 kernel on the CUDA cores and (where the sizes allow it) the
    tensor-core kernel against the formula, on a ragged batch over scattered pages: a portion behind 300
    cached tokens, a portion from the start, and single rows far into their requests (their keys shared
    out over several blocks)."""
    import numpy as np

    from mini_llm_runtime_b200.ops.cuda_ops import AttentionBatch, plan_attention

    k = ops.current()
    generator = torch.Generator().manual_seed(heads * 100 + dim)
    lengths, starts = np.array([70, 33, 1, 1], dtype=np.int32), np.array([300, 0, 777, 64], dtype=np.int32)
    page, pages_per_request = 16, 50
    order = torch.randperm(4 * pages_per_request, generator=generator).to(torch.int32)
    table = order.view(4, pages_per_request)
    keys = torch.randn(4, 800, kv_heads, dim, generator=generator)
    keys = keys / keys.pow(2).mean(-1, keepdim=True).sqrt()
    values = torch.randn(4, 800, kv_heads, vdim, generator=generator)
    rows = int(lengths.sum())
    q = torch.randn(rows, heads, dim, generator=generator)
    q = q / q.pow(2).mean(-1, keepdim=True).sqrt()
    r1, r2 = torch.rand(heads, generator=generator), torch.rand(heads, generator=generator)
    pb = torch.randn(heads, generator=generator) - 2.0
    talk = torch.eye(heads) + 0.3 * torch.randn(heads, heads, generator=generator)
    scale = 2.0 / math.sqrt(dim)
    row_start = np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.int32)
    arrays, counts = plan_attention(lengths, starts)

    def dev(a, dtype=torch.int32):
        return torch.as_tensor(a).to(device=DEVICE, dtype=dtype).contiguous()

    batch = AttentionBatch(dev(row_start), dev(lengths), dev(starts), dev(np.arange(4)), dev(table), 4, int(lengths.max()),
                           int((starts + lengths).max()), {n: dev(v) for n, v in arrays.items()}, counts)
    for dtype, use_mma, limit in ((F32, False, 2e-5), (BF16, False, 1.5e-2), (BF16, True, 1.5e-2)):
        k_pool = torch.zeros(4 * pages_per_request, kv_heads, page, dim, dtype=dtype)
        v_pool = torch.zeros(4 * pages_per_request, kv_heads, page, vdim, dtype=dtype)
        for request in range(4):
            for position in range(800):
                at = int(table[request, position // page])
                k_pool[at, :, position % page] = keys[request, position].to(dtype)
                v_pool[at, :, position % page] = values[request, position].to(dtype)
        qd = q.to(dtype)
        k.use_mma_sigmoid = use_mma
        try:
            got = k.sigmoid_attention(qd.view(rows, -1).to(DEVICE), k_pool.to(DEVICE), v_pool.to(DEVICE), batch, heads, kv_heads,
                                      dim, vdim, scale, distance=(r1.to(DEVICE), r2.to(DEVICE)), score_bias=pb.to(DEVICE),
                                      head_mix=talk.to(DEVICE))
        finally:
            k.use_mma_sigmoid = True
        group = heads // kv_heads
        for request in range(4):
            for r in range(int(lengths[request])):
                position = int(starts[request]) + r
                kk = keys[request, :position + 1].to(dtype).double().repeat_interleave(group, dim=1)
                vv = values[request, :position + 1].to(dtype).double().repeat_interleave(group, dim=1)
                row = int(row_start[request]) + r
                score = torch.einsum("hd,khd->hk", qd[row].double(), kk) * scale
                distance = (position - torch.arange(position + 1)).double()
                score = score - r1.double()[:, None] * torch.log1p(r2.double()[:, None] * distance[None]) + pb.double()[:, None]
                want = torch.einsum("hk,khd->hd", talk.double() @ torch.sigmoid(score), vv).reshape(-1)
                error = float((got[row].double().cpu() - want).abs().max()) / float(want.abs().max())
                assert error < limit, f"{dtype}, tensor cores {use_mma}: request {request}, row {r}: off by {error:.2e}"


def test_state_space_kernels_against_their_formulas():
    """Convolution, recurrence and gated norm on a ragged batch (a long portion, a single token, a
    portion shorter than the taps), then the same requests continued: the carried inputs and the state."""
    k = ops.current()
    generator = torch.Generator().manual_seed(5)
    heads, vdim, n, groups, taps, parts = 4, 12, 21, 2, 4, 2
    inner, gn = heads * vdim, groups * n
    channels = inner + 2 * gn
    width = 2 * inner + 2 * gn + heads
    conv = torch.randn(channels, taps, generator=generator) * 0.5
    conv_bias = torch.randn(channels, generator=generator) * 0.2
    dt_bias, a_log, skip = torch.randn(heads, generator=generator) * 0.5, torch.rand(heads, generator=generator) * 3 - 2.5, torch.randn(heads, generator=generator)
    weight = 1 + 0.2 * torch.randn(inner, generator=generator)
    lengths = [[37, 1, 2], [1, 3, 40]]
    total = [sum(col) for col in zip(*lengths)]
    sequences = [torch.randn(t, width, generator=generator) for t in total]
    conv_state = torch.zeros(3, taps - 1, channels, device=DEVICE)
    state = torch.zeros(3, heads, vdim, n, device=DEVICE)
    done = [0, 0, 0]
    got = [[], [], []]
    for step in lengths:
        rows = torch.cat([sequences[i][done[i]:done[i] + step[i]] for i in range(3)]).to(DEVICE)
        starts = [0, step[0], step[0] + step[1]]
        ctx = SimpleNamespace(seg_q_start=torch.tensor(starts, dtype=torch.int32, device=DEVICE),
                              seg_q_len=torch.tensor(step, dtype=torch.int32, device=DEVICE),
                              seg_slot=torch.tensor([2, 0, 1], dtype=torch.int32, device=DEVICE), num_segments=3, max_q_len=max(step))
        mixed = k.causal_conv(rows[:, inner:inner + channels], conv.to(DEVICE), conv_bias.to(DEVICE), conv_state, ctx, "silu")
        y = k.state_space_scan(mixed[:, :inner], mixed[:, inner:inner + gn], mixed[:, inner + gn:], rows[:, inner + channels:],
                               dt_bias.to(DEVICE), a_log.to(DEVICE), skip.to(DEVICE), state, ctx, heads, vdim, n, groups)
        out = k.gated_group_norm(y, rows[:, :inner], weight.to(DEVICE), 1e-5, parts, F32)
        for i in range(3):
            got[i].append(out[starts[i]:starts[i] + step[i]].cpu())
            done[i] += step[i]
    for i in range(3):
        u = sequences[i].double()
        xbc = plain.causal_conv_silu(u[:, inner:inner + channels], conv.double(), conv_bias.double())
        x, B, C = xbc[:, :inner].view(-1, heads, vdim), xbc[:, inner:inner + gn].view(-1, groups, n), xbc[:, inner + gn:].view(-1, groups, n)
        dt = torch.nn.functional.softplus(u[:, inner + channels:] + dt_bias.double())
        y = torch.zeros(total[i], heads, vdim, dtype=F64)
        for h in range(heads):
            S = torch.zeros(n, vdim, dtype=F64)
            for t in range(total[i]):
                S = torch.exp(-torch.exp(a_log[h].double()) * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, h // 2], x[t, h])
                y[t, h] = S.T @ C[t, h // 2] + skip[h].double() * x[t, h]
        y = y.reshape(total[i], inner) * plain.silu(u[:, :inner])
        want = plain.rms(y.view(total[i], parts, inner // parts), 1e-5).reshape(total[i], inner) * weight.double()
        assert float((torch.cat(got[i]).double() - want).abs().max()) < 2e-5 * float(want.abs().max()), f"request {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["MIXED", "ODD", "PLAIN"])
def test_prefill_against_token_by_token(name, dtype):
    config = getattr(rs, name)
    engine = rs.REngine(config, dtype, DEVICE, seed=1)
    tokens = rs.tokens_for(config["vocab"], 75, 8)
    want = engine.plain(tokens)
    rs.assert_logits_close(engine.run_cuts("whole", tokens, []), want, dtype, "whole")
    rs.assert_logits_close(engine.run_cuts("single", tokens, range(1, 75)), want, dtype, "token by token")
    rs.assert_logits_close(engine.run_cuts("tail", tokens, [40] + list(range(41, 75))), want, dtype, "prompt then decode")


@pytest.mark.parametrize("cuts", [[2, 4, 6, 8], [3, 19, 20, 52], [16, 32, 48, 64], [1, 2, 35, 37, 90], [17, 34, 51]])
def test_portions_of_several_sizes(cuts):
    engine = rs.REngine(rs.MIXED, F32, DEVICE, seed=4)
    tokens = rs.tokens_for(131, 100, 9)
    rs.assert_logits_close(engine.run_cuts("a", tokens, cuts), engine.plain(tokens), F32)


def test_float32_logits_do_not_depend_on_the_cut():
    engine = rs.REngine(rs.MIXED, F32, DEVICE, seed=4)
    tokens = rs.tokens_for(131, 90, 10)
    whole = engine.run_cuts("a", tokens, [])
    pieces = engine.run_cuts("b", tokens, [2, 5, 30, 31, 64])
    assert float((whole - pieces).abs().max()) <= 2e-5 * float(whole.abs().max())


def test_the_first_tokens_of_a_sequence():
    engine = rs.REngine(rs.MIXED, F32, DEVICE, seed=6)
    for length in (1, 2, 3, 13):
        tokens = rs.tokens_for(131, length, length)
        want = engine.plain(tokens)
        rs.assert_logits_close(engine.run_cuts("p", tokens, []), want, F32, f"prompt of {length}")
        rs.assert_logits_close(engine.run_cuts("d", tokens, range(1, length)), want, F32, f"decoded from the first token, {length}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_batches_of_unequal_requests(dtype):
    engine = rs.REngine(rs.MIXED, dtype, DEVICE, seed=6, num_pages=40)
    prompts = {"a": rs.tokens_for(131, 70, 1), "b": rs.tokens_for(131, 41, 2), "c": rs.tokens_for(131, 9, 3),
               "d": rs.tokens_for(131, 100, 4)}
    plan = [{"a": 30, "b": 1, "d": 2}, {"a": 1, "b": 16, "c": 9, "d": 50}, {"a": 1, "b": 1, "d": 1},
            {"a": 38, "b": 23, "d": 47}]
    got = engine.run_plan(prompts, plan)
    for name, tokens in prompts.items():
        rs.assert_logits_close(got[name], engine.plain(tokens), dtype, name)


def test_pages_and_slots_are_used_again():
    """Two slots and few pages serve six requests in turn: a slot's state and carried inputs start at
    zero again, and pages written by one request are read by the next."""
    config = rs.config([rs.parallel(rs.heads(2, 1, 8, 12), (2, 4, 6, 2, 3, 1), rs.moe(24, 4, 2, groups=(2, 1), shared=8)),
                        rs.attention(4, 2, 6, 4, v_mix=True), rs.attention(2, 2, 10, 4, v_mix=True, mlp=rs.dense(12))],
                       width=40, vocab=70)
    slow = {"l0.mix.right.A_log": lambda t: torch.full_like(t, -5.0)}       # a state left behind would stay for long
    engine = rs.REngine(config, F32, DEVICE, seed=3, page_size=8, num_pages=[14, 14, 14], max_requests=2, max_tokens=64,
                        max_step_tokens=16, overrides=slow)
    for number in range(3):
        prompts = {f"a{number}": rs.tokens_for(70, 33 + 7 * number, 20 + number), f"b{number}": rs.tokens_for(70, 25, 30 + number)}
        plan = []
        for start in range(0, 60, 6):
            step = {name: min(6, len(tokens) - start) for name, tokens in prompts.items() if start < len(tokens)}
            if step:
                plan.append(step)
        got = engine.run_plan(prompts, plan)
        for name, tokens in prompts.items():
            rs.assert_logits_close(got[name], engine.plain(tokens), F32, name)
        engine.cache.check_consistency()
    assert engine.cache.stats().free_pages == (14, 14, 14)


@pytest.mark.parametrize("how", ["prompt", "decoded", "portions"])
@pytest.mark.parametrize("query,key", [
    (290, 2),       # a key far back among hundreds
    (271, 15),      # far back, at the last place of a page
    (64, 63),       # the neighbour, across a page's border
    (48, 32),       # a page's first place
    (5, 0),         # the very first token
])
def test_far_keys_and_page_borders_with_a_dominant_key(query, key, how):
    length = 300
    config, overrides = rs.dominant_key_case(length, query, key, seed=query + key)
    engine = rs.REngine(config, F32, DEVICE, seed=5, overrides=overrides, num_pages=24, max_tokens=320)
    tokens = list(range(length))
    want = engine.plain(tokens)
    cuts = {"prompt": [], "decoded": [3] + list(range(4, length)), "portions": [2, max(3, query - 1), query, query + 2]}[how]
    got = engine.run_cuts("a", tokens, cuts)
    rs.assert_logits_close(got[query:query + 1], want[query:query + 1], F32, f"query {query}")
    rs.assert_logits_close(got, want, F32)
    # the case tells: with another token at the key's place, the answer at the query differs
    hidden = list(tokens)
    hidden[key] = (key + 101) % length
    other = engine.plain(hidden)
    assert float((other[query] - want[query]).abs().max()) > 1e-2 * float(want[query].abs().max())


@pytest.mark.parametrize("how", ["prompt", "decoded"])
@pytest.mark.parametrize("query,key", [
    (599, 511),     # the last key of the first 512: the end of a block's share of a long row
    (599, 512),     # the first key of the next share
    (590, 2),       # far back among hundreds
    (530, 479),     # across a key tile's border
])
def test_far_keys_through_the_tensor_core_kernel(query, key, how):
    """The same with heads of 64 in bfloat16, which the tensor-core kernel takes: a prompt of 600 tokens
    is shared out over blocks in chunks of keys, decoded rows in smaller ones."""
    length = 600
    config, overrides = rs.dominant_key_case(length, query, key, seed=query + key, dim=64, vdim=64, kv_heads=2)
    engine = rs.REngine(config, BF16, DEVICE, seed=5, overrides=overrides, num_pages=40, max_tokens=640)
    tokens = list(range(length))
    want = engine.plain(tokens)
    cuts = {"prompt": [], "decoded": [520] + list(range(521, length))}[how]
    got = engine.run_cuts("a", tokens, cuts)
    rs.assert_logits_close(got[query:query + 1], want[query:query + 1], BF16, f"query {query}")
    rs.assert_logits_close(got, want, BF16)
    hidden = list(tokens)
    hidden[key] = (key + 101) % length
    other = engine.plain(hidden)
    assert float((other[query] - want[query]).abs().max()) > 0.1 * float(want[query].abs().max())


def test_the_distance_bias_counts_from_the_right_end():
    """A distance bias strong enough that only the nearest keys count: a distance that is one off, or
    taken from the wrong end, changes the answer."""
    config = rs.config([rs.attention(2, 1, 8, 8, scale=0.1)], width=24, vocab=50)
    strong = {"l0.mix.r1": lambda t: torch.full_like(t, 6.0), "l0.mix.r2": lambda t: torch.full_like(t, 2.0),
              "l0.mix.pb": lambda t: torch.full_like(t, 2.0)}
    engine = rs.REngine(config, F32, DEVICE, seed=9, overrides=strong)
    tokens = rs.tokens_for(50, 140, 4)
    want = engine.plain(tokens)
    rs.assert_logits_close(engine.run_cuts("a", tokens, []), want, F32, "whole")
    rs.assert_logits_close(engine.run_cuts("b", tokens, [100] + list(range(101, 140))), want, F32, "decoded")
    changed = list(tokens)
    changed[120] = (changed[120] + 7) % 50
    other = engine.plain(changed)
    assert float((other[121] - want[121]).abs().max()) > 5e-3 * float(want[121].abs().max())      # the neighbour counts
    assert float((other[139] - want[139]).abs().max()) < 1e-2 * float(want[139].abs().max())      # 19 back hardly does


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_through_captured_steps(dtype):
    engine = rs.REngine(rs.MIXED, dtype, DEVICE, seed=12, num_pages=64)
    tokens = rs.tokens_for(131, 260, 13)
    want = engine.plain(tokens)
    got = engine.run_cuts("a", tokens, [30] + list(range(31, 260)))
    assert engine.runner.graph_replays > 100
    rs.assert_logits_close(got, want, dtype)
    other = rs.tokens_for(131, 60, 14)
    engine.cache.create_request("x")
    engine.cache.create_request("y")
    first = engine.step([("x", tokens[:20], range(20)), ("y", other[:10], range(10))])
    rows = {"x": [first[:20]], "y": [first[20:]]}
    for i in range(40):
        logits = engine.step([("x", tokens[20 + i:21 + i], [0]), ("y", other[10 + i:11 + i], [0])])
        rows["x"].append(logits[:1])
        rows["y"].append(logits[1:])
    rs.assert_logits_close(torch.cat(rows["x"]), rs.take(want, slice(0, 60)), dtype, "x")
    rs.assert_logits_close(torch.cat(rows["y"]), engine.plain(other[:50]), dtype, "y")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_the_tensor_core_kernels_take(dtype):
    engine = rs.REngine(rs.WIDE, dtype, DEVICE, seed=21, num_pages=80, max_tokens=1024)
    tokens = rs.tokens_for(520, 420, 22)
    want = engine.plain(tokens)
    rs.assert_logits_close(engine.run_cuts("a", tokens, [300, 301, 302, 350]), want, dtype)
    prompts = {"p": tokens[:200], "q": rs.tokens_for(520, 150, 24)}
    got = engine.run_plan(prompts, [{"p": 130, "q": 1}, {"p": 1, "q": 140}, {"p": 69, "q": 9}])
    rs.assert_logits_close(got["p"], rs.take(want, slice(0, 200)), dtype, "p")
    rs.assert_logits_close(got["q"], engine.plain(prompts["q"]), dtype, "q")


@pytest.mark.parametrize("seed", range(4))
def test_configurations_drawn_at_random(seed):
    config = rs.random_config(seed + 100)
    engine = rs.REngine(config, F32, DEVICE, seed=seed, num_pages=40)
    prompts = {"a": rs.tokens_for(config["vocab"], 45, seed), "b": rs.tokens_for(config["vocab"], 21, seed + 50)}
    got = engine.run_plan(prompts, [{"a": 17, "b": 1}, {"a": 1, "b": 2}, {"a": 2, "b": 18}, {"a": 25}])
    for name, tokens in prompts.items():
        rs.assert_logits_close(got[name], engine.plain(tokens), F32, f"seed {seed} {name}")


def test_greedy_generation_through_the_scheduler():
    parts = rs.REngine(rs.MIXED, F32, DEVICE, seed=31)
    engine = ContinuousBatchEngine.from_model(parts.model, block_size=8, total_blocks=96, max_running_requests=3,
                                              max_batch_tokens=24, max_model_len=160)
    prompts = [rs.tokens_for(131, length, 40 + i) for i, length in enumerate([5, 37, 18, 50, 2])]
    generated = engine.generate(prompts, max_new_tokens=12)
    for prompt, got in zip(prompts, generated):
        sequence = list(prompt)
        for _ in range(12):
            sequence.append(int(torch.argmax(parts.plain(sequence)[-1])))
        assert got == sequence[len(prompt):]


def test_command_line_and_replay_program_with_a_model_folder(tmp_path):
    """``make-random`` writes a Ratilorn folder from a config.json, ``generate`` reproduces the plain
    implementation's greedy tokens from it, and the replay program writes the logits of the wanted
    places step by step, with pages and slots given back in between."""
    import os
    import subprocess
    import sys

    import numpy as np

    from mini_llm_runtime_b200.weights import read_checkpoint

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))

    def cli(*arguments, stdin=None):
        done = subprocess.run([sys.executable, *arguments], capture_output=True, text=True, env=env, timeout=600,
                              input=stdin)
        assert done.returncode == 0, done.stderr[-2000:]
        return done.stdout

    (tmp_path / "config.json").write_text(json.dumps(rs.MIXED))
    folder = tmp_path / "model"
    cli("-m", "mini_llm_runtime_b200", "make-random", "--config", str(tmp_path / "config.json"), "--seed", "4",
        "--out", str(folder))
    tensors = read_checkpoint(folder)
    prompt = rs.tokens_for(131, 11, 6)
    sequence = list(prompt)
    for _ in range(5):
        sequence.append(int(torch.argmax(plain.forward(rs.MIXED, tensors, sequence)[0][-1])))
    record = json.loads(cli("-m", "mini_llm_runtime_b200", "generate", "--model", str(folder), "--dtype", "float32",
                            "--max-model-len", "64", "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "5"
                            ).splitlines()[-1])
    assert record["generated_ids"] == sequence[len(prompt):]

    other = rs.tokens_for(131, 30, 7)
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": prompt[:4], "want": [0, 3]}], "end": []},
             {"step": 1, "entries": [{"id": "p", "tokens": prompt[4:], "want": [6]},
                                     {"id": "o", "tokens": other, "want": [29]}], "end": ["p"]},
             {"step": 2, "entries": [], "end": ["o"]}]
    out = cli(os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out",
              str(tmp_path / "logits"), "--max-tokens", "64", stdin="\n".join(json.dumps(s) for s in steps) + "\n")
    assert [line for line in out.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    first = torch.from_numpy(np.fromfile(tmp_path / "logits" / "0.f32", dtype="<f4").reshape(2, 131))
    second = torch.from_numpy(np.fromfile(tmp_path / "logits" / "1.f32", dtype="<f4").reshape(2, 131))
    want = plain.forward(rs.MIXED, tensors, prompt)[0]
    rs.assert_logits_close(torch.cat([first, second[:1]]), want[[0, 3, 10]], F32)
    rs.assert_logits_close(second[1:], plain.forward(rs.MIXED, tensors, other)[0][29:], F32)
