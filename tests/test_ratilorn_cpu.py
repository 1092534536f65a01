"""Ratilorn's host side without a GPU: configuration and registry, weight names, cache needs, the
oracle's own mechanisms, and the whole engine (step function, scheduler) on the stand-in kernels
against the plain implementation."""

from __future__ import annotations

import json
import math

import pytest
import torch

import plain_ratilorn as plain
import ratilorn_support as rs
from fake_ops import FakeOps
from mini_llm_runtime_b200 import ops
from mini_llm_runtime_b200.config import RatilornConfig, config_from_dict, load_config
from mini_llm_runtime_b200.engine import ContinuousBatchEngine
from mini_llm_runtime_b200.models import build_model, write_random_model_dir
from mini_llm_runtime_b200.parts import KVCacheNeed, StateNeed
from mini_llm_runtime_b200.weights.loader import WeightError

F32 = torch.float32
F64 = torch.float64


def test_config_round_trip_and_registry(tmp_path):
    config = config_from_dict(rs.MIXED)
    assert isinstance(config, RatilornConfig) and config.vocab_size == 131 and len(config.layers) == 5
    assert config_from_dict(config.to_dict()) == config
    assert config.to_dict() == rs.MIXED
    assert config_from_dict(rs.PLAIN).to_dict() == rs.PLAIN
    folder = write_random_model_dir(tmp_path / "model", config, seed=3)
    entry, loaded = load_config(folder)
    assert entry.name == "Ratilorn" and loaded == config
    stored = json.loads((folder / "config.json").read_text())
    assert stored["layers"][1]["mlp"]["router"]["groups"] == {"count": 3, "keep": 2} and stored["layers"][2]["mlp"] is None
    assert stored["layers"][1]["mlp"]["shared"] == {"ff": 16} and "shared" not in stored["layers"][3]["mlp"]
    assert stored["layers"][3]["mixer"]["right"]["norm_groups"] == 2 and stored["layers"][1]["mixer"]["v_mix"] is True


@pytest.mark.parametrize("damage,message", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(groups=2), "groups"),
    (lambda c: c["layers"][3]["mixer"]["right"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(conv=1), "conv"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c.update(layers=[]), "layer"),
])
def test_config_errors(damage, message):
    data = json.loads(json.dumps(rs.MIXED))
    damage(data)
    with pytest.raises((KeyError, ValueError), match=message):
        config_from_dict(data)


def test_expected_tensors_and_cache_needs():
    model = build_model(config_from_dict(rs.MIXED), F32)
    expected = model.expected_tensors()
    assert expected["embed"].shape == (131, 96) and expected["pos"].shape == (512, 96) and "head" not in expected
    assert expected["l0.mix.left.q"].shape == (64, 96) and expected["l0.mix.left.k.b"].shape == (32,)
    assert expected["l0.mix.left.v"].shape == (48, 96) and expected["l0.mix.left.o"].shape == (96, 96)
    assert expected["l0.mix.left.q.norm"].shape == (16,) and expected["l0.mix.left.out"].shape == (96,)
    # in-projection: z and x of heads * vdim each, B and C of groups * state each, one dt per head
    assert expected["l0.mix.right.in"].shape == (2 * 24 + 2 * 20 + 3, 96) and expected["l0.mix.right.conv"].shape == (24 + 40, 4)
    assert expected["l3.mix.right.in"].shape == (2 * 24 + 2 * 2 * 18 + 4, 96) and expected["l3.mix.right.conv"].shape == (24 + 72, 2)
    assert expected["l0.mix.right.A_log"].shape == (3,) and expected["l0.mix.right.norm"].shape == (24,)
    assert expected["l1.mix.talk"].shape == (6, 6) and expected["l1.mix.r1"].shape == (6,) and expected["l1.mix.vmix"].shape == ()
    assert "l2.mix.vmix" not in expected and "l1.mix.q.norm" not in expected and "l2.norm2" not in expected
    assert expected["l1.mlp.shared.gate"].shape == (16, 96) and "l3.mlp.shared.gate" not in expected
    assert expected["l0.mlp.gate"].shape == (40, 96) and expected["l3.mlp.e7.down"].shape == (96, 32)
    needs = model.cache_needs()
    assert needs[0] == (KVCacheNeed(2, 16, None, value_dim=24), StateNeed((3, 8, 20), F32, "state"), StateNeed((3, 64), F32, "conv"))
    assert needs[1] == KVCacheNeed(2, 12, None, value_dim=8) and needs[2] == KVCacheNeed(3, 8, None, value_dim=12)
    assert build_model(config_from_dict(rs.PLAIN), F32).cache_needs()[1] == KVCacheNeed(2, 16, None)
    tensors = rs.draw_tensors(expected, 1)
    del tensors["l1.mlp.correction"]
    tensors["l0.mix.right.D"] = torch.zeros(5, dtype=torch.bfloat16)
    with ops.use(FakeOps()), pytest.raises(WeightError) as error:
        build_model(config_from_dict(rs.MIXED), F32).load(tensors, "cpu")
    assert "l1.mlp.correction" in error.value.missing and error.value.wrong_shape[0][0] == "l0.mix.right.D"


def test_the_oracles_router():
    """The grouped choice by hand: sigmoid scores, a correction that enters the choice only, groups
    ranked by the SUM of their two best choice scores, the others counting as minus infinity although
    choice scores are negative, weights renormalised."""
    t = {"r.router": torch.eye(6, dtype=F64), "r.correction": torch.tensor([0.0, -0.9, -0.3, -0.3, -0.95, -0.2], dtype=F64)}
    h = torch.tensor([[3.0, -3.0, 1.0, 1.0, 0.0, 0.5]], dtype=F64)
    s = torch.sigmoid(h[0])
    # groups (0,1), (2,3), (4,5): the largest single choice score is expert 0's (0.95), but group 1's two
    # (0.43 + 0.43) beat group 0's (0.95 - 0.85) and group 2's (-0.45 + 0.42)
    chosen, weights, _ = plain.route(h, t, "r.", {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert sorted(chosen.tolist()[0]) == [2, 3] and math.isclose(float(weights.sum()), 1.0)
    assert torch.allclose(weights[0], s[chosen[0]] / s[chosen[0]].sum())
    chosen, _, _ = plain.route(h, t, "r.", {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}})
    assert sorted(chosen.tolist()[0]) == [0, 2, 3]      # group 0 is second; expert 1 (-0.85) loses inside the kept groups
    chosen, _, _ = plain.route(h, t, "r.", {"experts": 6, "top": 3})
    assert sorted(chosen.tolist()[0]) == [0, 2, 3]
    with ops.use(FakeOps()) as fake:
        got, got_weights = fake.route_experts(h.float(), t["r.router"].float(), t["r.correction"].float(), 2, 3, 1, "sigmoid",
                                              True, group_top=2, renorm_eps=1e-20)
    assert sorted(got.tolist()[0]) == [2, 3] and math.isclose(float(got_weights.sum()), 1.0, rel_tol=1e-6)


def test_each_mechanism_shows_in_the_oracle():
    """The oracle's answer changes visibly when a mechanism is altered."""
    with ops.use(FakeOps()):
        engine = rs.REngine(rs.MIXED, F32, "cpu", seed=2)
    tokens = rs.tokens_for(131, 50, 3)
    want = engine.plain(tokens)

    def differs(config_dict=None, tensors=None):
        other, _ = plain.forward(config_dict or rs.MIXED, tensors or engine.tensors, tokens)
        return float((other - want).abs().max()) > 1e-3 * float(want.abs().max())

    def changed(edit):
        data = json.loads(json.dumps(rs.MIXED))
        edit(data)
        return data

    def tensor(name, edit):
        return {**engine.tensors, name: edit(engine.tensors[name].float()).to(torch.bfloat16)}

    assert differs(changed(lambda c: c["layers"][1]["mixer"].pop("v_mix")))        # then layer 4 is the first and blends nothing
    assert differs(changed(lambda c: c["layers"][1]["mixer"].update(scale=0.1)))
    assert differs(changed(lambda c: c["layers"][1]["mlp"]["router"].update(groups={"count": 3, "keep": 1})))
    assert differs(changed(lambda c: c["layers"][3]["mlp"]["router"].pop("groups")))
    assert differs(changed(lambda c: c["layers"][3]["mixer"]["right"].update(norm_groups=1)))
    assert differs(changed(lambda c: c.update(logit_scale=1.0)))
    for name in ("l1.mix.r1", "l1.mix.r2", "l1.mix.pb", "l4.mix.vmix", "l0.mix.right.A_log", "l0.mix.right.dt_bias",
                 "l0.mix.right.D", "l0.mix.right.conv.b", "l0.mix.left.q.norm", "l0.mix.right.out", "pos"):
        assert differs(tensors=tensor(name, lambda v: v * 1.5 + 0.25)), name
    assert differs(tensors=tensor("l1.mlp.correction", lambda v: v.flip(0) * 8))
    assert differs(tensors=tensor("l1.mix.talk", lambda v: v.T.contiguous()))
    assert differs(tensors=tensor("l0.mix.right.conv", lambda v: v.flip(1)))
    assert not differs(tensors=tensor("l1.mix.vmix", lambda v: v * 3))             # the first blending layer's own number is unused
    # norm weights are stored as offsets from one: zeros mean "times one", not "times zero"
    x = torch.randn(3, 8, dtype=F64)
    assert torch.allclose(plain.one_plus_norm(x, torch.zeros(8, dtype=F64), 1e-6), plain.rms(x, 1e-6))
    # sigmoid weights are not normalised: doubling the visible keys about doubles a head's output
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.0}
    t = {"a.q": torch.zeros(4, 4), "a.k": torch.zeros(4, 4), "a.v": torch.zeros(4, 4), "a.o": torch.eye(4), "a.q.b": torch.ones(4),
         "a.k.b": torch.ones(4), "a.v.b": torch.ones(4), "a.r1": torch.zeros(1), "a.r2": torch.ones(1), "a.pb": torch.zeros(1),
         "a.talk": torch.ones(1, 1)}
    out, _ = plain.sigmoid_attention(torch.zeros(6, 4, dtype=F64), t, "a.", m, 1e-6)
    assert torch.allclose(out[:, 0], 0.5 * torch.arange(1, 7, dtype=F64))


def test_the_convolution_and_the_state_are_carried():
    """The state-space layer cut anywhere equals the layer run whole (the stand-in kernels keep the last
    inputs of the convolution and the state per request)."""
    config = rs.config([rs.parallel(rs.heads(2, 1, 8, 8), (2, 6, 9, 1, 4, 1))], width=24, vocab=30)
    with ops.use(FakeOps()):
        engine = rs.REngine(config, F32, "cpu", seed=5, overrides={"l0.mix.right.A_log": lambda t: torch.full_like(t, -4.0)})
        tokens = rs.tokens_for(30, 40, 1)
        want = engine.plain(tokens)
        for cuts in ([], [1], [2, 3, 4], [1, 2, 3, 4, 5, 6], range(1, 40), [3, 20, 22]):
            rs.assert_logits_close(engine.run_cuts("r", tokens, cuts), want, F32, f"cuts {list(cuts)[:4]}")


@pytest.mark.parametrize("name", ["MIXED", "ODD", "PLAIN"])
def test_whole_prompt_token_by_token_and_portions(name):
    config = getattr(rs, name)
    with ops.use(FakeOps()):
        engine = rs.REngine(config, F32, "cpu", seed=1)
        tokens = rs.tokens_for(config["vocab"], 60, 8)
        want = engine.plain(tokens)
        rs.assert_logits_close(engine.run_cuts("whole", tokens, []), want, F32, "whole")
        rs.assert_logits_close(engine.run_cuts("single", tokens, range(1, 60)), want, F32, "token by token")
        rs.assert_logits_close(engine.run_cuts("cut", tokens, [2, 4, 21, 22, 50]), want, F32, "portions")


def test_batches_pages_and_slots_used_again():
    config = rs.config([rs.parallel(rs.heads(2, 1, 8, 12), (2, 4, 6, 2, 3, 1), rs.moe(24, 4, 2, groups=(2, 1), shared=8)),
                        rs.attention(4, 2, 6, 4, v_mix=True), rs.attention(2, 2, 10, 4, v_mix=True, mlp=rs.dense(12))],
                       width=40, vocab=70)
    with ops.use(FakeOps()):
        engine = rs.REngine(config, F32, "cpu", seed=3, page_size=8, num_pages=[14, 14, 14], max_requests=2, max_tokens=64,
                            max_step_tokens=16)
        for number in range(3):
            prompts = {f"a{number}": rs.tokens_for(70, 33 + 7 * number, 20 + number),
                       f"b{number}": rs.tokens_for(70, 25, 30 + number)}
            plan = []
            for start in range(0, 60, 6):
                step = {name: min(6, len(tokens) - start) for name, tokens in prompts.items() if start < len(tokens)}
                if step:
                    plan.append(step)
            got = engine.run_plan(prompts, plan)
            for name, tokens in prompts.items():
                rs.assert_logits_close(got[name], engine.plain(tokens), F32, name)
            engine.cache.check_consistency()
        assert engine.cache.stats().free_pages == (14, 14, 14) and engine.cache.stats().free_slots == 2


def test_greedy_generation_through_the_scheduler():
    with ops.use(FakeOps()):
        parts = rs.REngine(rs.MIXED, F32, "cpu", seed=31)
        engine = ContinuousBatchEngine.from_model(parts.model, block_size=8, total_blocks=96, max_running_requests=3,
                                                  max_batch_tokens=24, max_model_len=120)
        prompts = [rs.tokens_for(131, length, 40 + i) for i, length in enumerate([5, 37, 18, 2])]
        generated = engine.generate(prompts, max_new_tokens=6)
    for prompt, got in zip(prompts, generated):
        sequence = list(prompt)
        for _ in range(6):
            sequence.append(int(torch.argmax(parts.plain(sequence)[-1])))
        assert got == sequence[len(prompt):]


@pytest.mark.parametrize("seed", range(6))
def test_configurations_drawn_at_random(seed):
    config = rs.random_config(seed)
    with ops.use(FakeOps()):
        engine = rs.REngine(config, F32, "cpu", seed=seed, num_pages=40)
        prompts = {"a": rs.tokens_for(config["vocab"], 45, seed), "b": rs.tokens_for(config["vocab"], 21, seed + 50)}
        got = engine.run_plan(prompts, [{"a": 17, "b": 1}, {"a": 1, "b": 2}, {"a": 2, "b": 18}, {"a": 25}])
    for name, tokens in prompts.items():
        rs.assert_logits_close(got[name], engine.plain(tokens), F32, f"seed {seed} {name}")
