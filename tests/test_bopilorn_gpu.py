"""Bopilorn through the framework's model, cache manager, step function and kernels, against the
plain implementation (``plain_bopilorn``): each mechanism alone, whole prompts, token-by-token
decoding, portions, mixed batches, reused pages and slots, far keys and page borders with a key made
to dominate, the first tokens, long decoding through captured steps, odd and larger sizes, and greedy
generation through the scheduler and the command line."""

from __future__ import annotations

import json
import math

import pytest
import torch

import bopilorn_support as bs
import plain_bopilorn as plain
from mini_llm_runtime_b200.engine import ContinuousBatchEngine

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
F32 = torch.float32
BF16 = torch.bfloat16
DTYPES = [torch.float32, torch.bfloat16]


def one_layer(mlp=None, **options):
    return bs.config([bs.attention(6, 2, 16, 24, mlp=mlp, **options)], width=72, vocab=90, embedding_scale=1.7)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("options", [{}, {"dims": 10}, {"scaling": (4.0, 32.0, 8.0, 1.0)}, {"base": 50.0, "scale": 0.6}])
def test_the_mixer_alone(options, dtype):
    engine = bs.BEngine(one_layer(**options), dtype, DEVICE, seed=11)
    tokens = bs.tokens_for(90, 61, 5)
    bs.assert_logits_close(engine.run_cuts("a", tokens, []), engine.plain(tokens), dtype, "whole")
    bs.assert_logits_close(engine.run_cuts("b", tokens, [30] + list(range(31, 61))), engine.plain(tokens), dtype, "decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mlp", [bs.moe(56, 6, 2), bs.moe(56, 6, 3, groups=(3, 2)), bs.moe(40, 8, 2, groups=(4, 1)),
                                 bs.moe(64, 3, 1), bs.moe(24, 2, 2, groups=(1, 1))])
def test_the_feed_forward(mlp, dtype):
    tokens = bs.tokens_for(90, 40, 3)
    engine = bs.BEngine(one_layer(mlp=mlp), dtype, DEVICE, seed=2)
    bs.assert_logits_close(engine.run_cuts("a", tokens, [25, 26]), engine.plain(tokens), dtype)


def test_router_kernel_against_its_formula():
    from mini_llm_runtime_b200 import ops
    k = ops.current()
    generator = torch.Generator().manual_seed(5)
    for rows, width, experts, top, groups, keep in [(1, 40, 6, 2, 3, 1), (37, 68, 12, 4, 4, 2), (9, 96, 5, 5, 1, 1),
                                                    (130, 24, 64, 6, 8, 3), (3, 33, 7, 1, 7, 2)]:
        x = torch.randn(rows, width, generator=generator)
        router = torch.randn(experts, width, generator=generator) * 0.5
        correction = torch.randn(experts, generator=generator) * 0.3 - 0.4        # mostly negative choice scores
        t = {"m.router": router.double(), "m.correction": correction.double()}
        want_chosen, want_weights = plain.route(x.double(), t, "m.", {"experts": experts, "top": top,
                                                                     "groups": {"count": groups, "keep": keep}})
        chosen, weights = k.route_experts(x.to(DEVICE), router.to(DEVICE), correction.to(DEVICE), top, groups, keep)
        assert chosen.cpu().tolist() == want_chosen.tolist()
        assert torch.allclose(weights.cpu().double(), want_weights, rtol=1e-5, atol=1e-7)
        half = k.route_experts(x.to(DEVICE).to(BF16), router.to(DEVICE), correction.to(DEVICE), top, groups, keep)[1]
        assert half.shape == weights.shape
    # renormalised weights and sigmoid scores are parameters of the same kernel
    chosen, weights = k.route_experts(x.to(DEVICE), router.to(DEVICE), None, 1, 1, 1, "sigmoid", True)
    assert torch.allclose(weights.cpu(), torch.ones(3, 1))
    assert chosen.cpu().flatten().tolist() == (x @ router.T).argmax(-1).tolist()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width,inner,experts,top", [(1, 40, 24, 3, 2), (5, 72, 52, 5, 1), (150, 64, 64, 4, 3),
                                                            (300, 128, 192, 8, 2), (700, 256, 128, 16, 4), (20, 36, 20, 2, 2),
                                                            (700, 512, 256, 4, 2), (900, 768, 384, 5, 3)])
def test_expert_kernels_against_their_formula(rows, width, inner, experts, top, dtype):
    """Few and many rows (the sorted, grouped tensor-core product takes the latter in bfloat16: in tiles
    of 128 rows of an expert, or of 256 where the products are wide and the experts get many rows),
    sizes with and without the interleaved gate/up blocks, experts that get no row at all."""
    from mini_llm_runtime_b200 import ops
    from mini_llm_runtime_b200.config import PartSpec
    from mini_llm_runtime_b200.parts import build_part
    generator = torch.Generator().manual_seed(rows)
    part = build_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": width, "intermediate_size": inner, "experts": experts, "top": top}, "m."), dtype)
    tensors = bs.draw_tensors(part.tensors(), rows)
    part.load(tensors, DEVICE)
    x = torch.randn(rows, width, generator=generator).to(BF16)
    pool = experts - 1 if experts > top else experts      # where there is room, the last expert stays idle
    chosen = torch.stack([torch.randperm(pool, generator=generator)[:top] for _ in range(rows)]).to(torch.int32)
    weights = torch.rand(rows, top, generator=generator)
    kernels = ops.current()
    before = kernels.use_tall_expert_tiles
    kernels.use_tall_expert_tiles = rows == 900          # one of the wide cases in tiles of 256 rows
    try:
        got = kernels.routed_experts(x.to(DEVICE).to(dtype), chosen.to(DEVICE), weights.to(DEVICE), part.w_gate_up,
                                     part.w_down, part.block)
    finally:
        kernels.use_tall_expert_tiles = before
    want = torch.zeros(rows, width, dtype=torch.float64)
    x64 = x.double()
    for e in range(experts):
        gate, up, down = (tensors[f"m.e{e}.{n}"].double() for n in ("gate", "up", "down"))
        hidden = torch.nn.functional.silu(x64 @ gate.T) * (x64 @ up.T)
        if dtype == BF16:
            hidden = hidden.to(BF16).double()
        y = hidden @ down.T
        for t in range(top):
            mask = chosen[:, t] == e
            want[mask] += weights[mask, t, None].double() * y[mask]
    error = float((got.double().cpu() - want).abs().max()) / float(want.abs().max())
    assert error < (1e-5 if dtype == F32 else 1.5e-2), error


def test_grouped_and_plain_products_share_a_kernel_without_harm():
    """The grouped product and the plain product of many rows are launches of one kernel with rings
    of different depths; each keeps working after the other has run."""
    from mini_llm_runtime_b200 import ops
    k = ops.current()
    generator = torch.Generator().manual_seed(3)
    x = torch.randn(300, 1024, generator=generator).to(BF16).to(DEVICE)
    w = (torch.randn(1024, 1024, generator=generator) * 0.03).to(BF16).to(DEVICE)
    want = x.float() @ w.float().T
    small = torch.randn(300, 64, generator=generator).to(BF16).to(DEVICE)
    gate_up = (torch.randn(4, 256, 64, generator=generator) * 0.1).to(BF16).to(DEVICE)
    down = (torch.randn(4, 64, 128, generator=generator) * 0.1).to(BF16).to(DEVICE)
    chosen = torch.randint(0, 4, (300, 1), generator=generator, dtype=torch.int32).to(DEVICE)
    weights = torch.ones(300, 1, device=DEVICE)
    for _ in range(2):
        got = k.linear(x, w, out_dtype=F32)
        assert float((got - want).abs().max()) < 2e-2 * float(want.abs().max())
        assert torch.isfinite(k.routed_experts(small, chosen, weights, gate_up, down, 64)).all()
    torch.cuda.synchronize()
    k.raise_if_device_error()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot,interleaved", [(6, 2, 16, 24, 16, True), (3, 3, 10, 6, 6, True),
                                                                      (4, 1, 64, 64, 32, False), (2, 2, 128, 64, 128, True),
                                                                      (16, 4, 128, 128, 128, True), (32, 8, 128, 128, 64, True),
                                                                      (2, 1, 32, 16, 16, False), (2, 2, 16, 8, 4, True)])
def test_prepare_and_turn_kernels_against_their_formulas(heads, kv_heads, dim, vdim, rot, interleaved, dtype):
    from mini_llm_runtime_b200 import ops
    k = ops.current()
    generator = torch.Generator().manual_seed(dim)
    rows, page = 21, 8
    qkv = torch.randn(rows, (heads + kv_heads) * dim + kv_heads * vdim, generator=generator) * 2
    positions = torch.randint(0, 3000, (rows,), generator=generator, dtype=torch.int32)
    q_weight, k_weight = 1 + 0.3 * torch.randn(heads * dim, generator=generator), 1 + 0.3 * torch.randn(kv_heads * dim, generator=generator)
    rope = {"base": 1000.0, "dims": rot, "scaling": {"factor": 3.0, "original": 200.0, "fast": 16.0, "slow": 1.0}}
    key_freq, magnitude = plain.key_frequencies(rope)
    value_freq = plain.value_frequencies(1000.0, vdim)
    slots = torch.randperm(4 * page, generator=generator)[:rows].to(torch.int64)
    k_pool = torch.zeros(4, kv_heads, page, dim, dtype=dtype, device=DEVICE)
    v_pool = torch.zeros(4, kv_heads, page, vdim, dtype=dtype, device=DEVICE)
    dev = lambda t: t.to(DEVICE)      # noqa: E731
    q = k.rotated_prepare(dev(qkv), dev(positions), dev(q_weight), dev(k_weight), 1e-5, dev(torch.tensor(key_freq, dtype=F32)),
                          magnitude, dev(torch.tensor(value_freq, dtype=F32)), interleaved, True, dev(slots), k_pool, v_pool,
                          heads, kv_heads, dim, vdim)

    def turn(vector, frequencies, factor=1.0, sign=1.0):
        if interleaved:
            return plain.turn(vector, positions, frequencies, factor, sign)
        n = 2 * len(frequencies)      # pairs (i, i + n/2): bring them side by side, turn, and back
        order = torch.stack([torch.arange(n // 2), torch.arange(n // 2) + n // 2], dim=1).flatten()
        out = vector.clone()
        out[..., order] = plain.turn(vector[..., order], positions, frequencies, factor, sign)
        return out

    x = qkv.double()
    want_q = turn((plain.rms(x[:, :heads * dim], 1e-5) * q_weight).reshape(rows, heads, dim), key_freq, magnitude)
    want_k = turn((plain.rms(x[:, heads * dim:(heads + kv_heads) * dim], 1e-5) * k_weight).reshape(rows, kv_heads, dim),
                  key_freq, magnitude)
    want_v = turn(plain.rms(x[:, (heads + kv_heads) * dim:].reshape(rows, kv_heads, vdim), 1e-5), value_freq)
    limit = 2e-3 if dtype == F32 else 4e-2       # angles of positions in the thousands are 32-bit
    assert float((q.double().cpu().view(rows, heads, dim) - want_q).abs().max()) < limit * float(want_q.abs().max())
    stored_k = k_pool.double().cpu().permute(0, 2, 1, 3).reshape(4 * page, kv_heads, dim)[slots]
    stored_v = v_pool.double().cpu().permute(0, 2, 1, 3).reshape(4 * page, kv_heads, vdim)[slots]
    assert float((stored_k - want_k).abs().max()) < limit * float(want_k.abs().max())
    assert float((stored_v - want_v).abs().max()) < limit * float(want_v.abs().max())
    # the way back: turning the stored values by minus their positions gives the normalised values again
    heads_of_values = want_v.to(dtype).to(DEVICE).reshape(rows, kv_heads * vdim).contiguous()
    back = k.turn_heads(heads_of_values, dev(positions), dev(torch.tensor(value_freq, dtype=F32)), kv_heads, vdim,
                        interleaved, sign=-1.0)
    unturned = plain.rms(x[:, (heads + kv_heads) * dim:].reshape(rows, kv_heads, vdim), 1e-5)
    assert float((back.double().cpu().view(rows, kv_heads, vdim) - unturned).abs().max()) < limit * 4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["MIXED", "ODD", "PLAIN"])
def test_prefill_against_token_by_token(name, dtype):
    config = getattr(bs, name)
    engine = bs.BEngine(config, dtype, DEVICE, seed=1)
    tokens = bs.tokens_for(config["vocab"], 75, 8)
    want = engine.plain(tokens)
    bs.assert_logits_close(engine.run_cuts("whole", tokens, []), want, dtype, "whole")
    bs.assert_logits_close(engine.run_cuts("single", tokens, range(1, 75)), want, dtype, "token by token")
    bs.assert_logits_close(engine.run_cuts("tail", tokens, [40] + list(range(41, 75))), want, dtype, "prompt then decode")


@pytest.mark.parametrize("cuts", [[2, 4, 6, 8], [3, 19, 20, 52], [16, 32, 48, 64], [1, 2, 35, 37, 90], [17, 34, 51]])
def test_portions_of_several_sizes(cuts):
    engine = bs.BEngine(bs.MIXED, F32, DEVICE, seed=4)
    tokens = bs.tokens_for(131, 100, 9)
    bs.assert_logits_close(engine.run_cuts("a", tokens, cuts), engine.plain(tokens), F32)


def test_float32_logits_do_not_depend_on_the_cut():
    engine = bs.BEngine(bs.MIXED, F32, DEVICE, seed=4)
    tokens = bs.tokens_for(131, 90, 10)
    whole = engine.run_cuts("a", tokens, [])
    pieces = engine.run_cuts("b", tokens, [2, 5, 30, 31, 64])
    assert float((whole - pieces).abs().max()) <= 2e-5 * float(whole.abs().max())


def test_the_first_tokens_of_a_sequence():
    engine = bs.BEngine(bs.MIXED, F32, DEVICE, seed=6)
    for length in (1, 2, 3, 13):
        tokens = bs.tokens_for(131, length, length)
        want = engine.plain(tokens)
        bs.assert_logits_close(engine.run_cuts("p", tokens, []), want, F32, f"prompt of {length}")
        bs.assert_logits_close(engine.run_cuts("d", tokens, range(1, length)), want, F32, f"decoded from the first token, {length}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_batches_of_unequal_requests(dtype):
    engine = bs.BEngine(bs.MIXED, dtype, DEVICE, seed=6, num_pages=40)
    prompts = {"a": bs.tokens_for(131, 70, 1), "b": bs.tokens_for(131, 41, 2), "c": bs.tokens_for(131, 9, 3),
               "d": bs.tokens_for(131, 100, 4)}
    plan = [{"a": 30, "b": 1, "d": 2}, {"a": 1, "b": 16, "c": 9, "d": 50}, {"a": 1, "b": 1, "d": 1},
            {"a": 38, "b": 23, "d": 47}]
    got = engine.run_plan(prompts, plan)
    for name, tokens in prompts.items():
        bs.assert_logits_close(got[name], engine.plain(tokens), dtype, name)


def test_pages_and_slots_are_used_again():
    config = bs.config([bs.attention(2, 1, 8, 12, mlp=bs.moe(24, 4, 2, groups=(2, 1))), bs.attention(4, 2, 6, 4, dims=4)],
                       width=40, vocab=70, embedding_scale=1.3)
    engine = bs.BEngine(config, F32, DEVICE, seed=3, page_size=8, num_pages=[14, 14], max_requests=2, max_tokens=64,
                        max_step_tokens=16)
    for number in range(3):
        prompts = {f"a{number}": bs.tokens_for(70, 33 + 7 * number, 20 + number), f"b{number}": bs.tokens_for(70, 25, 30 + number)}
        plan = []
        for start in range(0, 60, 6):
            step = {name: min(6, len(tokens) - start) for name, tokens in prompts.items() if start < len(tokens)}
            if step:
                plan.append(step)
        got = engine.run_plan(prompts, plan)
        for name, tokens in prompts.items():
            bs.assert_logits_close(got[name], engine.plain(tokens), F32, name)
        engine.cache.check_consistency()
    assert engine.cache.stats().free_pages == (14, 14)


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
    config, overrides = bs.dominant_key_case(length, query, key, seed=query + key)
    engine = bs.BEngine(config, F32, DEVICE, seed=5, overrides=overrides, num_pages=24, max_tokens=320)
    tokens = list(range(length))
    want = engine.plain(tokens)
    cuts = {"prompt": [], "decoded": [3] + list(range(4, length)), "portions": [2, max(3, query - 1), query, query + 2]}[how]
    got = engine.run_cuts("a", tokens, cuts)
    bs.assert_logits_close(got[query:query + 1], want[query:query + 1], F32, f"query {query}")
    bs.assert_logits_close(got, want, F32)
    # the case tells: with another token at the key's place, the answer at the query differs
    hidden = list(tokens)
    hidden[key] = (key + 101) % length
    other = engine.plain(hidden)
    assert float((other[query] - want[query]).abs().max()) > 1e-2 * float(want[query].abs().max())
    # and so does the way back of the values' rotation: turned by a neighbour's angle, the answer is another
    original = plain.turn

    def one_off(vector, positions, frequencies, magnitude=1.0, sign=1.0):
        return original(vector, positions + 1 if sign < 0 else positions, frequencies, magnitude, sign)

    plain.turn = one_off
    try:
        shifted = engine.plain(tokens)
    finally:
        plain.turn = original
    assert float((shifted[query] - want[query]).abs().max()) > 1e-2 * float(want[query].abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_through_captured_steps(dtype):
    engine = bs.BEngine(bs.MIXED, dtype, DEVICE, seed=12, num_pages=64)
    tokens = bs.tokens_for(131, 260, 13)
    want = engine.plain(tokens)
    got = engine.run_cuts("a", tokens, [30] + list(range(31, 260)))
    assert engine.runner.graph_replays > 100
    bs.assert_logits_close(got, want, dtype)
    other = bs.tokens_for(131, 60, 14)
    engine.cache.create_request("x")
    engine.cache.create_request("y")
    first = engine.step([("x", tokens[:20], range(20)), ("y", other[:10], range(10))])
    rows = {"x": [first[:20]], "y": [first[20:]]}
    for i in range(40):
        logits = engine.step([("x", tokens[20 + i:21 + i], [0]), ("y", other[10 + i:11 + i], [0])])
        rows["x"].append(logits[:1])
        rows["y"].append(logits[1:])
    bs.assert_logits_close(torch.cat(rows["x"]), bs.take(want, slice(0, 60)), dtype, "x")
    bs.assert_logits_close(torch.cat(rows["y"]), engine.plain(other[:50]), dtype, "y")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_the_tensor_core_kernels_take(dtype):
    engine = bs.BEngine(bs.WIDE, dtype, DEVICE, seed=21, num_pages=80, max_tokens=1024)
    tokens = bs.tokens_for(520, 420, 22)
    want = engine.plain(tokens)
    bs.assert_logits_close(engine.run_cuts("a", tokens, [300, 301, 302, 350]), want, dtype)
    prompts = {"p": tokens[:200], "q": bs.tokens_for(520, 150, 23)}
    got = engine.run_plan(prompts, [{"p": 130, "q": 1}, {"p": 1, "q": 140}, {"p": 69, "q": 9}])
    bs.assert_logits_close(got["p"], bs.take(want, slice(0, 200)), dtype, "p")
    bs.assert_logits_close(got["q"], engine.plain(prompts["q"]), dtype, "q")


@pytest.mark.parametrize("seed", range(4))
def test_configurations_drawn_at_random(seed):
    config = bs.random_config(seed + 100)
    engine = bs.BEngine(config, F32, DEVICE, seed=seed, num_pages=40)
    prompts = {"a": bs.tokens_for(config["vocab"], 45, seed), "b": bs.tokens_for(config["vocab"], 21, seed + 50)}
    got = engine.run_plan(prompts, [{"a": 17, "b": 1}, {"a": 1, "b": 2}, {"a": 2, "b": 18}, {"a": 25}])
    for name, tokens in prompts.items():
        bs.assert_logits_close(got[name], engine.plain(tokens), F32, f"seed {seed} {name}")


def test_greedy_generation_through_the_scheduler():
    parts = bs.BEngine(bs.MIXED, F32, DEVICE, seed=31)
    engine = ContinuousBatchEngine.from_model(parts.model, block_size=8, total_blocks=96, max_running_requests=3,
                                              max_batch_tokens=24, max_model_len=160)
    prompts = [bs.tokens_for(131, length, 40 + i) for i, length in enumerate([5, 37, 18, 50, 2])]
    generated = engine.generate(prompts, max_new_tokens=12)
    for prompt, got in zip(prompts, generated):
        sequence = list(prompt)
        for _ in range(12):
            sequence.append(int(torch.argmax(parts.plain(sequence)[-1])))
        assert got == sequence[len(prompt):]


def test_command_line_and_replay_program_with_a_model_folder(tmp_path):
    """``make-random`` writes a Bopilorn folder from a config.json, ``generate`` reproduces the plain
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

    (tmp_path / "config.json").write_text(json.dumps(bs.MIXED))
    folder = tmp_path / "model"
    cli("-m", "mini_llm_runtime_b200", "make-random", "--config", str(tmp_path / "config.json"), "--seed", "4",
        "--out", str(folder))
    tensors = read_checkpoint(folder)
    prompt = bs.tokens_for(131, 11, 6)
    sequence = list(prompt)
    for _ in range(5):
        sequence.append(int(torch.argmax(plain.forward(bs.MIXED, tensors, sequence)[-1])))
    record = json.loads(cli("-m", "mini_llm_runtime_b200", "generate", "--model", str(folder), "--dtype", "float32",
                            "--max-model-len", "64", "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "5"
                            ).splitlines()[-1])
    assert record["generated_ids"] == sequence[len(prompt):]

    other = bs.tokens_for(131, 30, 7)
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": prompt[:4], "want": [0, 3]}], "end": []},
             {"step": 1, "entries": [{"id": "p", "tokens": prompt[4:], "want": [6]},
                                     {"id": "o", "tokens": other, "want": [29]}], "end": ["p"]},
             {"step": 2, "entries": [], "end": ["o"]}]
    out = cli(os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out",
              str(tmp_path / "logits"), "--max-tokens", "64", stdin="\n".join(json.dumps(s) for s in steps) + "\n")
    assert [line for line in out.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    first = torch.from_numpy(np.fromfile(tmp_path / "logits" / "0.f32", dtype="<f4").reshape(2, 131))
    second = torch.from_numpy(np.fromfile(tmp_path / "logits" / "1.f32", dtype="<f4").reshape(2, 131))
    want = plain.forward(bs.MIXED, tensors, prompt)
    bs.assert_logits_close(torch.cat([first, second[:1]]), want[[0, 3, 10]], F32)
    bs.assert_logits_close(second[1:], plain.forward(bs.MIXED, tensors, other)[29:], F32)
