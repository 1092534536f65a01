"""Rozesun through the framework's model, cache manager, step function and kernels, against the
plain implementation (``plain_rozesun``): each mechanism alone, whole prompts, token-by-token
decoding, portions, mixed batches, reused pages and slots, window edges and far keys with a key made
to dominate, the first tokens, long decoding through captured steps, odd and larger sizes, and greedy
generation through the scheduler and the command line."""

from __future__ import annotations

import json
import math

import pytest
import torch

import plain_rozesun as plain
import rozesun_support as rs
from mini_llm_runtime_b200.engine import ContinuousBatchEngine

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
F32 = torch.float32
DTYPES = [torch.float32, torch.bfloat16]


def one_layer(kind, ff=0):
    layer = (rs.latent2(3, 16, 8, 40, 24, 20, window=9, ff=ff) if kind == "latent_attention_2"
             else rs.latent(3, 16, 8, 40, 24, 20, ff=ff))
    return rs.config([layer], width=72, vocab=90, logit_scale=1.2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["latent_attention", "latent_attention_2"])
def test_each_mixer_alone(kind, dtype):
    engine = rs.REngine(one_layer(kind), dtype, DEVICE, seed=11)
    tokens = rs.tokens_for(90, 61, 5)
    rs.assert_logits_close(engine.run_cuts("a", tokens, []), engine.plain(tokens), dtype, kind)
    rs.assert_logits_close(engine.run_cuts("b", tokens, [30] + list(range(31, 61))), engine.plain(tokens), dtype, kind)


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_and_loop_vectors(dtype):
    tokens = rs.tokens_for(90, 25, 3)
    engine = rs.REngine(one_layer("latent_attention", ff=56), dtype, DEVICE, seed=2)
    rs.assert_logits_close(engine.run_cuts("a", tokens, []), engine.plain(tokens), dtype)
    looped = {**one_layer("latent_attention_2", ff=56), "loop": {"start": 0, "stop": 1, "times": 3}}
    engine = rs.REngine(looped, dtype, DEVICE, seed=2)
    rs.assert_logits_close(engine.run_cuts("a", tokens, [11]), engine.plain(tokens), dtype)


def test_kernels_against_their_formulas():
    from mini_llm_runtime_b200 import ops
    k = ops.current()
    generator = torch.Generator().manual_seed(5)
    for rows, width in [(1, 40), (7, 68), (33, 1000), (3, 5000), (70, 5000), (5, 4096), (70, 4096), (2, 2052), (9, 8192), (4, 8196)]:
        x = torch.randn(rows, width, generator=generator) * 3 + 1
        delta = torch.randn(rows, width, generator=generator) * 2
        vectors = [torch.randn(width, generator=generator) for _ in range(5)]
        dw, db, offset, w, b = vectors
        want_x = x.double() + plain.layer_norm(delta.double(), dw.double(), db.double(), 1e-5) + offset.double()
        want = plain.layer_norm(want_x, w.double(), b.double(), 1e-5)
        stream = x.to(DEVICE)
        got = k.layer_norm_step(stream, 1e-5, delta=delta.to(DEVICE), delta_norm=(dw.to(DEVICE), db.to(DEVICE)),
                                offset=offset.to(DEVICE), norm=(w.to(DEVICE), b.to(DEVICE)), out_dtype=F32)
        assert float((stream.double().cpu() - want_x).abs().max()) < 1e-5
        assert float((got.double().cpu() - want).abs().max()) < 1e-4
        only = k.layer_norm_step(x.to(DEVICE), 1e-5, norm=(w.to(DEVICE), b.to(DEVICE)), out_dtype=torch.bfloat16)
        assert float((only.double().cpu() - plain.layer_norm(x.double(), w.double(), b.double(), 1e-5)).abs().max()) < 0.05
    gate_up = torch.randn(9, 2 * 48, generator=generator) * 2
    blocks = gate_up.view(9, 3, 2, 16)
    g, u = blocks[:, :, 0].reshape(9, 48).clamp(max=0.9), blocks[:, :, 1].reshape(9, 48).clamp(-0.9, 0.9)
    got = k.clamped_gate(gate_up.to(DEVICE), 16, 0.9, 1.702)
    assert float((got.cpu() - g * torch.sigmoid(1.702 * g) * (u + 1)).abs().max()) < 1e-6


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
    config = rs.config([rs.latent2(2, 8, 4, 8, 12, 8, window=20, ff=24, limit=1.0), rs.latent(2, 8, 8, 4, 8, 12)],
                       width=40, vocab=70, loop=(0, 2, 2), logit_scale=1.3)
    engine = rs.REngine(config, F32, DEVICE, seed=3, page_size=8, num_pages=[14, 40], max_requests=2, max_tokens=160,
                        max_step_tokens=16)
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
    assert engine.cache.stats().free_pages == (14, 40)
    tokens = rs.tokens_for(70, 150, 77)
    got = engine.run_cuts("long", tokens, list(range(10, 150, 10)), release=False)
    windowed = engine.cache.get("long").pages[0]
    assert windowed[0] < 0 and sum(p >= 0 for p in windowed) <= 5
    rs.assert_logits_close(got, engine.plain(tokens), F32, "long")


@pytest.mark.parametrize("how", ["prompt", "decoded", "portions"])
@pytest.mark.parametrize("kind,window,query,key", [
    ("latent_attention_2", 10, 40, 31),     # just inside the window
    ("latent_attention_2", 10, 40, 30),     # just outside
    ("latent_attention_2", 16, 47, 32),     # a window's edge on a page's border
    ("latent_attention_2", 16, 48, 32),     # and one past it
    ("latent_attention_2", 33, 290, 258),   # the window's last key, far into the sequence
    ("latent_attention", 0, 290, 2),        # a key far back among hundreds
    ("latent_attention", 0, 271, 15),       # far back, at the last place of a page
    ("latent_attention", 0, 64, 63),        # the neighbour, across a page's border
])
def test_edges_and_far_keys_with_a_dominant_key(kind, window, query, key, how):
    length = 300
    config, overrides = rs.dominant_key_case(kind, window, length, query, key, seed=query + key)
    engine = rs.REngine(config, F32, DEVICE, seed=5, overrides=overrides, num_pages=24, max_tokens=320)
    tokens = list(range(length))
    want = engine.plain(tokens)
    cuts = {"prompt": [], "decoded": [20] + list(range(21, length)), "portions": [7, query - 1, query, query + 2]}[how]
    got = engine.run_cuts("a", tokens, cuts)
    rs.assert_logits_close(got[query:query + 1], want[query:query + 1], F32, f"query {query}")
    rs.assert_logits_close(got, want, F32)
    # the case tells: were the key hidden (or, outside the window, seen), the answer at the query would differ
    if kind == "latent_attention_2":
        inside = plain.sees(query, key, window)
        moved = json.loads(json.dumps(config))
        moved["layers"][0]["mixer"]["mask"]["size"] = window + (-1 if inside and query - key == window - 1 else 1)
        other = engine.plain(tokens, moved)
    else:
        hidden = list(tokens)
        hidden[key] = (key + 101) % length
        other = engine.plain(hidden)
    assert float((other[query] - want[query]).abs().max()) > 1e-2 * float(want[query].abs().max())


def test_a_sink_takes_its_share():
    config, overrides = rs.dominant_key_case("latent_attention_2", 10, 60, 40, 35, seed=3)
    overrides["l0.mix.sink"] = lambda t: torch.tensor([6.0, -2.0])
    engine = rs.REngine(config, F32, DEVICE, seed=5, overrides=overrides)
    tokens = list(range(60))
    want = engine.plain(tokens)
    rs.assert_logits_close(engine.run_cuts("a", tokens, [50, 51]), want, F32)
    without = plain.forward(config, {**engine.tensors, "l0.mix.sink": torch.tensor([-40.0, -40.0])}, tokens)
    assert float((without - want).abs().max()) > 1e-2 * float(want.abs().max())


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
    rs.assert_logits_close(torch.cat(rows["x"]), want[:60], dtype, "x")
    rs.assert_logits_close(torch.cat(rows["y"]), engine.plain(other[:50]), dtype, "y")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_the_tensor_core_products_take(dtype):
    engine = rs.REngine(rs.WIDE, dtype, DEVICE, seed=21, num_pages=80, max_tokens=1024)
    tokens = rs.tokens_for(520, 420, 22)
    want = engine.plain(tokens)
    rs.assert_logits_close(engine.run_cuts("a", tokens, [300, 301, 302, 350]), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_large_latent_and_many_heads(dtype):
    """A latent of 512 with a turned part of 64 (the largest the attention kernels hold) under 18
    heads (more than one group of the decode kernel, the last one short)."""
    config = rs.config([rs.latent(18, 8, 64, 8, 512, 16, ff=32), rs.latent2(5, 8, 2, 8, 200, 16, window=40)],
                       width=64, vocab=60, logit_scale=0.5)
    engine = rs.REngine(config, dtype, DEVICE, seed=8)
    tokens = rs.tokens_for(60, 90, 4)
    want = engine.plain(tokens)
    rs.assert_logits_close(engine.run_cuts("a", tokens, []), want, dtype, "whole")
    rs.assert_logits_close(engine.run_cuts("b", tokens, [70, 71, 72, 80]), want, dtype, "portions and single tokens")


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
    """``make-random`` writes a Rozesun folder from a config.json, ``generate`` reproduces the plain
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
        sequence.append(int(torch.argmax(plain.forward(rs.MIXED, tensors, sequence)[-1])))
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
    want = plain.forward(rs.MIXED, tensors, prompt)
    rs.assert_logits_close(torch.cat([first, second[:1]]), want[[0, 3, 10]], F32)
    rs.assert_logits_close(second[1:], plain.forward(rs.MIXED, tensors, other)[29:], F32)


def _attention_case(lengths, positions, heads, rank, rot, page=16, seed=0):
    """A ragged batch over a paged cache of random rows, as the attention kernels take it."""
    import numpy as np

    from mini_llm_runtime_b200.ops.cuda_ops import AttentionBatch, plan_attention

    generator = torch.Generator().manual_seed(seed)
    lengths, positions = np.asarray(lengths, dtype=np.int32), np.asarray(positions, dtype=np.int32)
    starts = np.zeros_like(lengths)
    np.cumsum(lengths[:-1], out=starts[1:])
    per_request = -(-int((positions + lengths).max()) // page)
    order = torch.randperm(len(lengths) * per_request, generator=generator).to(torch.int32)      # pages in any order
    table = order.view(len(lengths), per_request).to(DEVICE)
    pool = torch.randn(len(lengths) * per_request, 1, page, rank + rot, generator=generator).to(torch.bfloat16).to(DEVICE)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEVICE)      # noqa: E731
    arrays, counts = plan_attention(lengths, positions)
    batch = AttentionBatch(dev(starts), dev(lengths), dev(positions), dev(np.arange(len(lengths))), table, len(lengths),
                           int(lengths.max()), int((positions + lengths).max()), {n: dev(v) for n, v in arrays.items()}, counts)
    q = (torch.randn(int(lengths.sum()), heads * (rank + rot), generator=generator) * 0.3).to(torch.bfloat16).to(DEVICE)
    return q, pool, batch


@pytest.mark.parametrize("heads,rank,rot,window,sink", [(3, 40, 8, 0, False), (2, 88, 24, 37, True), (18, 64, 16, 100, True),
                                                         (16, 512, 64, 0, False), (1, 24, 8, 9, True)])
def test_tensor_core_attention_against_the_float32_kernel(heads, rank, rot, window, sink):
    """Prompt portions beside decoded rows (some in several key chunks) on the tensor-core kernels
    against the float32 kernels on the same bfloat16 rows."""
    from mini_llm_runtime_b200 import ops
    k = ops.current()
    q, pool, batch = _attention_case([70, 1, 33, 1, 1], [130, 299, 0, 40, 0], heads, rank, rot, seed=heads)
    sinks = torch.linspace(-1.0, 2.0, heads).to(DEVICE) if sink else None
    got = k.latent_attention(q, pool, batch, heads, rank, rot, 0.11, window, sinks)
    k.use_mma_attention = False
    try:
        want = k.latent_attention(q, pool, batch, heads, rank, rot, 0.11, window, sinks)
    finally:
        k.use_mma_attention = True
    assert float((got - want).abs().max()) < 2e-2 * float(want.abs().max())
    assert float((got - want).pow(2).mean().sqrt()) < 3e-3 * float(want.pow(2).mean().sqrt())


@pytest.mark.parametrize("rows", [1, 9, 150])
def test_per_head_products_against_the_formula(rows):
    from mini_llm_runtime_b200 import ops
    k = ops.current()
    generator = torch.Generator().manual_seed(rows)
    heads, dim, rot, rank, vdim = 3, 24, 8, 40, 16
    q = torch.randn(rows, heads * (dim + rot), generator=generator)
    w_uk = (torch.randn(heads * dim, rank, generator=generator) * 0.2).to(torch.bfloat16)
    positions = torch.arange(5, 5 + rows, dtype=torch.int32)
    frequencies = torch.tensor([1.0, 0.3, 0.02])        # three pairs: the last two of the eight entries pass unchanged
    for interleaved in (False, True):
        got = k.absorb_queries(q.to(DEVICE), w_uk.to(DEVICE), heads, dim, rot, rank, positions.to(DEVICE),
                               frequencies.to(DEVICE), interleaved).float().cpu().view(rows, heads, rank + rot)
        q3 = q.double().view(rows, heads, dim + rot)
        plain_part = torch.einsum("rhd,hdc->rhc", q3[..., :dim], w_uk.double().view(heads, dim, rank))
        turned = plain.rotate(q3[..., dim:], positions, 1.0, 6, interleaved)      # base 1: frequencies set below
        for i, f in enumerate(frequencies.tolist()):                              # the oracle's rotation with these angles
            a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + 3)
            angle = positions.double() * f
            u, v = q3[..., dim + a], q3[..., dim + b]
            turned[..., a] = u * torch.cos(angle)[:, None] - v * torch.sin(angle)[:, None]
            turned[..., b] = v * torch.cos(angle)[:, None] + u * torch.sin(angle)[:, None]
        want = torch.cat([plain_part, turned], dim=-1)
        assert float((got - want).abs().max()) < 2e-2 * float(want.abs().max())
    mixed = torch.randn(rows, heads * rank, generator=generator)
    w_uv = (torch.randn(heads * vdim, rank, generator=generator) * 0.2).to(torch.bfloat16)
    for per_head in (False, True):
        gate = torch.randn(rows, heads if per_head else heads * vdim, generator=generator)
        got = k.latent_values(mixed.to(DEVICE), w_uv.to(DEVICE), heads, vdim, rank, gate.to(DEVICE), per_head).float().cpu()
        want = torch.einsum("rhc,hvc->rhv", mixed.double().view(rows, heads, rank), w_uv.double().view(heads, vdim, rank))
        want = want * (torch.sigmoid(gate.double())[:, :, None] if per_head else torch.sigmoid(gate.double()).view(rows, heads, vdim))
        assert float((got.view(rows, heads, vdim) - want).abs().max()) < 2e-2 * float(want.abs().max())


@pytest.mark.parametrize("rows", [1, 8, 40, 130, 700])
@pytest.mark.parametrize("inner,width", [(256, 128), (1216, 896)])
def test_clamped_gate_product(rows, inner, width):
    """min(x Wg^T, c) * sigmoid(1.702 .) * (clamp(x Wu^T, -c, c) + 1) from the many-rows product's own
    epilogue and from the separate kernel behind the few-rows product, against the formula."""
    from mini_llm_runtime_b200 import ops

    generator = torch.Generator().manual_seed(rows + inner)
    x = torch.randn(rows, width, generator=generator).to(torch.bfloat16)
    gate = (torch.randn(inner, width, generator=generator) / width ** 0.5 * 2).to(torch.bfloat16)
    up = (torch.randn(inner, width, generator=generator) / width ** 0.5 * 2).to(torch.bfloat16)
    stacked = torch.cat([gate.view(-1, 64, width), up.view(-1, 64, width)], dim=1).reshape(2 * inner, width)
    got = ops.current().linear_clamped_gate(x.to(DEVICE), stacked.to(DEVICE).contiguous(), 64, 1.3, 1.702)
    g = (x.double() @ gate.double().T).clamp(max=1.3)
    u = (x.double() @ up.double().T).clamp(-1.3, 1.3)
    want = g * torch.sigmoid(1.702 * g) * (u + 1)
    assert float((got.double().cpu() - want).abs().max()) < 2e-2 * float(want.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed, dtype):
    """Layer kinds in any order, sizes of every parity, loops anywhere: a mixed batch and single tokens."""
    config = rs.random_config(seed)
    engine = rs.REngine(config, dtype, DEVICE, seed=seed, num_pages=40)
    prompts = {"a": rs.tokens_for(config["vocab"], 45, seed), "b": rs.tokens_for(config["vocab"], 21, seed + 50)}
    got = engine.run_plan(prompts, [{"a": 17, "b": 1}, {"a": 1, "b": 2}, {"a": 2, "b": 18}, {"a": 25}])
    for name, tokens in prompts.items():
        rs.assert_logits_close(got[name], engine.plain(tokens), dtype, f"seed {seed} {name}")
