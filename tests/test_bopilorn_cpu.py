"""Bopilorn's host side without a GPU: configuration and registry, weight names, cache needs, the
oracle's own mechanisms, and the whole engine (step function, scheduler) on the stand-in kernels
against the plain implementation."""

from __future__ import annotations

import json
import math

import pytest
import torch

import bopilorn_support as bs
import plain_bopilorn as plain
from fake_ops import FakeOps
from mini_llm_runtime_b200 import ops
from mini_llm_runtime_b200.config import BopilornConfig, PartSpec, config_from_dict, load_config
from mini_llm_runtime_b200.engine import ContinuousBatchEngine
from mini_llm_runtime_b200.models import build_model, write_random_model_dir
from mini_llm_runtime_b200.parts import KVCacheNeed, build_part
from mini_llm_runtime_b200.weights.loader import WeightError

F32 = torch.float32


def test_config_round_trip_and_registry(tmp_path):
    config = config_from_dict(bs.MIXED)
    assert isinstance(config, BopilornConfig) and config.vocab_size == 131 and len(config.layers) == 4
    assert config_from_dict(config.to_dict()) == config
    assert config.to_dict() == bs.MIXED
    assert config_from_dict(bs.PLAIN).to_dict() == bs.PLAIN      # a router without groups stays without
    folder = write_random_model_dir(tmp_path / "model", config, seed=3)
    entry, loaded = load_config(folder)
    assert entry.name == "Bopilorn" and loaded == config
    stored = json.loads((folder / "config.json").read_text())
    assert stored["layers"][0]["mlp"]["router"]["groups"] == {"count": 3, "keep": 2} and stored["layers"][2]["mlp"] is None
    assert stored["layers"][1]["mixer"]["rot"] == {"base": 500.0, "dims": 6}


@pytest.mark.parametrize("damage,message", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=2), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=7), "vdim"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=5), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "scaling"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("embedding"), "embedding"),
    (lambda c: c.update(layers=[]), "layer"),
])
def test_config_errors(damage, message):
    data = json.loads(json.dumps(bs.MIXED))
    damage(data)
    with pytest.raises((KeyError, ValueError), match=message):
        config_from_dict(data)


def test_expected_tensors_and_cache_needs():
    model = build_model(config_from_dict(bs.MIXED), F32)
    expected = model.expected_tensors()
    assert expected["embed"].shape == (131, 96) and expected["head"].shape == (131, 96) and expected["final.norm"].shape == (96,)
    assert expected["l0.mix.q"].shape == (64, 96) and expected["l0.mix.k"].shape == (32, 96)
    assert expected["l0.mix.v"].shape == (48, 96) and expected["l0.mix.o"].shape == (96, 96)
    assert expected["l0.mix.q.norm"].shape == (64,) and expected["l0.mix.k.norm"].shape == (32,)
    assert expected["l0.mlp.router"].shape == (6, 96) and expected["l0.mlp.correction"].shape == (6,)
    assert expected["l0.mlp.e5.gate"].shape == (40, 96) and expected["l0.mlp.e5.down"].shape == (96, 40)
    assert "l0.mlp.e6.gate" not in expected and "l2.mlp.router" not in expected and "l2.norm2" not in expected
    assert "l2.norm1b" in expected and not any(name.endswith(".b") for name in expected)
    assert model.cache_needs() == [KVCacheNeed(2, 16, None, value_dim=24), KVCacheNeed(3, 8, None, value_dim=12),
                                   KVCacheNeed(2, 12, None, value_dim=8), KVCacheNeed(1, 24, None, value_dim=16)]
    assert build_model(config_from_dict(bs.PLAIN), F32).cache_needs()[0] == KVCacheNeed(2, 16, None)
    tensors = bs.draw_tensors(expected, 1)
    del tensors["l0.mlp.correction"]
    tensors["l3.mix.k.norm"] = torch.zeros(5, dtype=torch.bfloat16)
    with ops.use(FakeOps()), pytest.raises(WeightError) as error:
        build_model(config_from_dict(bs.MIXED), F32).load(tensors, "cpu")
    assert "l0.mlp.correction" in error.value.missing and error.value.wrong_shape[0][0] == "l3.mix.k.norm"


def test_scaled_frequencies_of_the_position_part():
    """The position part's table against the oracle's, with and without the rescaling; a scaling whose
    ramp covers no pair, all pairs, and a part of them."""
    for dims, base, scaling in [(16, 10000.0, None), (16, 10000.0, (4.0, 64.0, 8.0, 1.0)), (6, 500.0, (2.5, 30.0, 4.0, 0.5)),
                                (64, 10000.0, (2.0, 2048.0, 32.0, 1.0)), (8, 50.0, (3.0, 1e6, 2.0, 1.0)),
                                (8, 50.0, (3.0, 4.0, 64.0, 32.0))]:
        rot = {"base": base, "dims": dims}
        args = {"head_dim": dims, "theta": base, "layout": "interleaved"}
        if scaling:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
            args["scaling"] = rot["scaling"]
        want, magnitude = plain.key_frequencies(rot)
        part = build_part("position", PartSpec("rope_pairs", args), F32)
        assert torch.allclose(part._inv_freq_cpu.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-6, atol=0)
        assert math.isclose(part.magnitude, magnitude, rel_tol=1e-12)
        if scaling:
            assert math.isclose(magnitude, 0.1 * math.log(scaling[0]) + 1.0)
    slowed, _ = plain.key_frequencies({"base": 8.0, "dims": 8, "scaling": {"factor": 4.0, "original": 16.0, "fast": 4.0, "slow": 1.0}})
    unscaled = [8.0 ** (-2.0 * i / 8) for i in range(4)]
    assert slowed[0] == unscaled[0] and math.isclose(slowed[3], unscaled[3] / 4.0) and unscaled[1] / 4.0 < slowed[1] < unscaled[1]


def test_the_oracles_router():
    """The grouped choice by hand: scores, the correction that enters the choice only, groups whose
    other experts count as minus infinity although choice scores are negative."""
    t = {"r.router": torch.eye(6, dtype=torch.float64) * 1.0, "r.correction": torch.tensor([0.0, -0.9, -0.8, -0.7, -0.95, -0.2], dtype=torch.float64)}
    h = torch.tensor([[2.0, 0.0, 0.0, 0.0, 1.0, 0.5]], dtype=torch.float64)
    scores = torch.softmax(h[0], dim=0)
    chosen, weights = plain.route(h, t, "r.", {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    # groups (0,1), (2,3), (4,5): group scores come from experts 0, 3 and 5; group 0 wins; its second
    # expert is taken although its choice score is far below those of the other groups
    assert chosen.tolist() == [[0, 1]] and torch.allclose(weights[0], scores[[0, 1]])
    chosen, weights = plain.route(h, t, "r.", {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}})
    assert chosen.tolist() == [[0, 5, 4]] and torch.allclose(weights[0], scores[[0, 5, 4]])
    chosen, _ = plain.route(h, t, "r.", {"experts": 6, "top": 3})
    assert chosen.tolist() == [[0, 5, 3]]
    assert float(weights.sum()) < 1.0     # not renormalised


def test_each_mechanism_shows_in_the_oracle():
    """The oracle's answer changes visibly when a mechanism is altered: the query/key norm's span, the
    frequency scaling, the value norm, the values' rotation and the way back, the groups, the
    correction, the embedding's scale."""
    with ops.use(FakeOps()):
        engine = bs.BEngine(bs.MIXED, F32, "cpu", seed=2)
    tokens = bs.tokens_for(131, 50, 3)
    want = engine.plain(tokens)

    def differs(config_dict=None, tensors=None):
        other = plain.forward(config_dict or bs.MIXED, tensors or engine.tensors, tokens)
        return float((other - want).abs().max()) > 1e-3 * float(want.abs().max())

    def changed(edit):
        data = json.loads(json.dumps(bs.MIXED))
        edit(data)
        return data

    assert differs(changed(lambda c: c["layers"][0]["mixer"]["rot"].pop("scaling")))
    assert differs(changed(lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(fast=2.0)))
    assert differs(changed(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=8)))
    assert differs(changed(lambda c: c["layers"][0]["mlp"]["router"].update(groups={"count": 3, "keep": 1})))
    assert differs(changed(lambda c: c["layers"][3]["mlp"]["router"].pop("groups")))
    assert differs(changed(lambda c: c["embedding"].update(scale=1.0)))
    assert differs(changed(lambda c: c["layers"][2]["mixer"].update(scale=0.1)))
    assert differs(tensors={**engine.tensors, "l0.mlp.correction": engine.tensors["l0.mlp.correction"].flip(0) * 4})
    # a per-head norm would not see this: one head's query weights doubled and another's halved
    weight = engine.tensors["l1.mix.q.norm"].clone()
    weight[:8] *= 2
    assert differs(tensors={**engine.tensors, "l1.mix.q.norm": weight})
    # values: scaling the value projection changes next to nothing (unit root mean square per head; eps)...
    same = plain.forward(bs.MIXED, {**engine.tensors, "l0.mix.v": engine.tensors["l0.mix.v"] * 2}, tokens)
    assert float((same - want).abs().max()) < 1e-4 * float(want.abs().max())
    # ...and the values' rotation is undone exactly when attention looks at the token itself only
    alone = plain.attention(torch.randn(1, 96, dtype=torch.float64), {k: v.double() for k, v in engine.tensors.items()},
                            "l0.mix.", bs.MIXED["layers"][0]["mixer"], 1e-5)
    assert alone.shape == (1, 96)
    original = plain.turn

    def no_way_back(vector, positions, frequencies, magnitude=1.0, sign=1.0):
        return vector.clone() if sign < 0 else original(vector, positions, frequencies, magnitude, sign)

    plain.turn = no_way_back
    try:
        assert differs()
    finally:
        plain.turn = original


@pytest.mark.parametrize("name", ["MIXED", "ODD", "PLAIN"])
def test_whole_prompt_token_by_token_and_portions(name):
    config = getattr(bs, name)
    with ops.use(FakeOps()):
        engine = bs.BEngine(config, F32, "cpu", seed=1)
        tokens = bs.tokens_for(config["vocab"], 60, 8)
        want = engine.plain(tokens)
        bs.assert_logits_close(engine.run_cuts("whole", tokens, []), want, F32, "whole")
        bs.assert_logits_close(engine.run_cuts("single", tokens, range(1, 60)), want, F32, "token by token")
        bs.assert_logits_close(engine.run_cuts("cut", tokens, [2, 4, 21, 22, 50]), want, F32, "portions")


def test_batches_pages_and_slots_used_again():
    config = bs.config([bs.attention(2, 1, 8, 12, mlp=bs.moe(24, 4, 2, groups=(2, 1))), bs.attention(4, 2, 6, 4, dims=4)],
                       width=40, vocab=70, embedding_scale=1.3)
    with ops.use(FakeOps()):
        engine = bs.BEngine(config, F32, "cpu", seed=3, page_size=8, num_pages=[14, 14], max_requests=2, max_tokens=64,
                            max_step_tokens=16)
        for number in range(3):
            prompts = {f"a{number}": bs.tokens_for(70, 33 + 7 * number, 20 + number),
                       f"b{number}": bs.tokens_for(70, 25, 30 + number)}
            plan = []
            for start in range(0, 60, 6):
                step = {name: min(6, len(tokens) - start) for name, tokens in prompts.items() if start < len(tokens)}
                if step:
                    plan.append(step)
            got = engine.run_plan(prompts, plan)
            for name, tokens in prompts.items():
                bs.assert_logits_close(got[name], engine.plain(tokens), F32, name)
            engine.cache.check_consistency()
        assert engine.cache.stats().free_pages == (14, 14) and engine.cache.stats().free_slots == 2


def test_greedy_generation_through_the_scheduler():
    with ops.use(FakeOps()):
        parts = bs.BEngine(bs.MIXED, F32, "cpu", seed=31)
        engine = ContinuousBatchEngine.from_model(parts.model, block_size=8, total_blocks=96, max_running_requests=3,
                                                  max_batch_tokens=24, max_model_len=120)
        prompts = [bs.tokens_for(131, length, 40 + i) for i, length in enumerate([5, 37, 18, 2])]
        generated = engine.generate(prompts, max_new_tokens=6)
    for prompt, got in zip(prompts, generated):
        sequence = list(prompt)
        for _ in range(6):
            sequence.append(int(torch.argmax(parts.plain(sequence)[-1])))
        assert got == sequence[len(prompt):]


@pytest.mark.parametrize("seed", range(6))
def test_configurations_drawn_at_random(seed):
    config = bs.random_config(seed)
    with ops.use(FakeOps()):
        engine = bs.BEngine(config, F32, "cpu", seed=seed, num_pages=40)
        prompts = {"a": bs.tokens_for(config["vocab"], 45, seed), "b": bs.tokens_for(config["vocab"], 21, seed + 50)}
        got = engine.run_plan(prompts, [{"a": 17, "b": 1}, {"a": 1, "b": 2}, {"a": 2, "b": 18}, {"a": 25}])
    for name, tokens in prompts.items():
        bs.assert_logits_close(got[name], engine.plain(tokens), F32, f"seed {seed} {name}")
