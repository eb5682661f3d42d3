"""Rozesun's host side without a GPU: configuration and registry, the looped run order, weight names,
the cache groups of windowed and full layers, and the whole engine (step function, scheduler, replay
program's loop) on the stand-in kernels against the plain implementation."""

from __future__ import annotations

import json

import pytest
import torch

import plain_rozesun as plain
import rozesun_support as rs
from fake_ops import FakeOps
from mini_llm_runtime_b200 import ops
from mini_llm_runtime_b200.config import RozesunConfig, config_from_dict, load_config
from mini_llm_runtime_b200.config.rozesun import rozesun_run_order
from mini_llm_runtime_b200.engine import ContinuousBatchEngine
from mini_llm_runtime_b200.models import build_model, write_random_model_dir
from mini_llm_runtime_b200.parts import KVCacheNeed
from mini_llm_runtime_b200.weights.loader import WeightError

F32 = torch.float32


def test_config_round_trip_and_registry(tmp_path):
    config = config_from_dict(rs.MIXED)
    assert isinstance(config, RozesunConfig) and config.vocab_size == 131 and len(config.layers) == 4
    assert config_from_dict(config.to_dict()) == config
    assert config.to_dict() == rs.MIXED
    assert config_from_dict(rs.PLAIN).to_dict() == rs.PLAIN            # no loop stays no loop
    folder = write_random_model_dir(tmp_path / "model", config, seed=3)
    entry, loaded = load_config(folder)
    assert entry.name == "Rozesun" and loaded == config
    stored = json.loads((folder / "config.json").read_text())
    assert stored["layers"][0]["mixer"]["mask"] == {"size": 12} and stored["loop"] == {"start": 1, "stop": 3, "times": 2}


@pytest.mark.parametrize("damage,message", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].pop("mask"), "mask"),
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=0), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=5), "dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "kind"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("logit_scale"), "logit_scale"),
    (lambda c: c.update(layers=[]), "layer"),
])
def test_config_errors(damage, message):
    data = json.loads(json.dumps(rs.MIXED))
    damage(data)
    with pytest.raises((KeyError, ValueError), match=message):
        config_from_dict(data)


def test_run_order_of_a_loop_and_its_cache_entries():
    order = rozesun_run_order(config_from_dict(rs.MIXED))
    assert [(s.layer, s.offset_row) for s in order] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert [s.cache for s in order] == list(range(6)) and all(s.writes_cache for s in order)
    assert [(s.layer, s.offset_row) for s in rozesun_run_order(config_from_dict(rs.ODD))] == [(0, 0)]
    assert [(s.layer, s.offset_row) for s in rozesun_run_order(config_from_dict(rs.PLAIN))] == [(0, None), (1, None)]
    assert [(s.layer, s.offset_row) for s in plain_order(rs.MIXED)] == [(s.layer, s.offset_row) for s in order]
    model = build_model(config_from_dict(rs.MIXED), F32)
    needs = model.cache_needs()
    assert needs[0] == KVCacheNeed(1, 48, 12, value_dim=0) and needs[1] == needs[3] == KVCacheNeed(1, 48, None, value_dim=0)
    assert needs[2] == needs[4] == KVCacheNeed(1, 32, None, value_dim=0) and needs[5] == KVCacheNeed(1, 20, 33, value_dim=0)


def plain_order(config_dict):
    from types import SimpleNamespace
    return [SimpleNamespace(layer=i, offset_row=n) for i, n in plain.run_order(config_dict)]


def test_expected_tensors():
    expected = build_model(config_from_dict(rs.MIXED), F32).expected_tensors()
    assert expected["embed"].shape == (131, 96) and expected["loop.step"].shape == (2, 96)
    assert expected["l0.mix.dq"].shape == (48, 96) and expected["l0.mix.uq"].shape == (3 * 24, 48)
    assert expected["l0.mix.dkv"].shape == (48, 96) and expected["l0.mix.dkv.norm"].shape == (40,)
    assert expected["l0.mix.uk"].shape == (48, 40) and expected["l0.mix.uv"].shape == (72, 40)
    assert expected["l0.mix.g"].shape == (3, 96) and expected["l0.mix.sink"].shape == (3,)
    assert expected["l1.mix.g"].shape == (64, 96) and "l1.mix.sink" not in expected
    assert "l2.mlp.gate" not in expected and "l2.norm2" not in expected and "l2.norm1b.b" in expected
    assert expected["final.norm.b"].shape == (96,) and "head" not in expected and "loop.step" not in \
        build_model(config_from_dict(rs.PLAIN), F32).expected_tensors()
    tensors = rs.draw_tensors(expected, 1)
    del tensors["l0.mix.sink"]
    tensors["l3.mix.g"] = torch.zeros(5, 96, dtype=torch.bfloat16)
    with ops.use(FakeOps()), pytest.raises(WeightError) as error:
        build_model(config_from_dict(rs.MIXED), F32).load(tensors, "cpu")
    assert "l0.mix.sink" in error.value.missing and error.value.wrong_shape[0][0] == "l3.mix.g"


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


def test_each_mechanism_shows_in_the_oracle():
    """The oracle's answer changes visibly when a mechanism is left out: the sink, the window's edge,
    the pair layout, the pass vectors, the clamp, the logit scale."""
    with ops.use(FakeOps()):
        engine = rs.REngine(rs.MIXED, F32, "cpu", seed=2)
    tokens = rs.tokens_for(131, 50, 3)
    want = engine.plain(tokens)

    def differs(config_dict=None, tensors=None):
        other = plain.forward(config_dict or rs.MIXED, tensors or engine.tensors, tokens)
        return float((other - want).abs().max()) > 1e-3 * float(want.abs().max())

    changed = json.loads(json.dumps(rs.MIXED))
    changed["layers"][0]["mixer"]["mask"]["size"] = 11
    assert differs(changed)
    changed = json.loads(json.dumps(rs.MIXED))
    changed["layers"][1]["mlp"]["limit"] = 0.6
    assert differs(changed)
    changed = json.loads(json.dumps(rs.MIXED))
    changed["layers"][0]["type"], changed["layers"][0]["mixer"]["mask"] = "latent_attention", None
    assert differs(changed, {**engine.tensors, "l0.mix.g": engine.tensors["l0.mix.g"].repeat_interleave(24, dim=0)})
    assert differs(tensors={**engine.tensors, "l0.mix.sink": engine.tensors["l0.mix.sink"] - 30.0})
    assert differs(tensors={**engine.tensors, "loop.step": engine.tensors["loop.step"].flip(0)})
    assert differs({**rs.MIXED, "logit_scale": 1.0})


def test_batches_pages_and_slots_used_again():
    # 2 slots, 14 pages of 8 per group: requests come and go, windowed layers give pages back while they run
    config = rs.config([rs.latent2(2, 8, 4, 8, 12, 8, window=20, ff=24, limit=1.0), rs.latent(2, 8, 8, 4, 8, 12)],
                       width=40, vocab=70, loop=(0, 2, 2), logit_scale=1.3)
    with ops.use(FakeOps()):
        engine = rs.REngine(config, F32, "cpu", seed=3, page_size=8, num_pages=[14, 40], max_requests=2, max_tokens=160,
                            max_step_tokens=16)
        for number in range(3):
            prompts = {f"a{number}": rs.tokens_for(70, 33 + 7 * number, 20 + number),
                       f"b{number}": rs.tokens_for(70, 25, 30 + number)}
            names = list(prompts)
            plan = []
            for start in range(0, 60, 6):
                step = {name: min(6, len(prompts[name]) - start) for name in names if start < len(prompts[name])}
                if step:
                    plan.append(step)
            got = engine.run_plan(prompts, plan)
            for name, tokens in prompts.items():
                rs.assert_logits_close(got[name], engine.plain(tokens), F32, name)
            engine.cache.check_consistency()
        assert engine.cache.stats().free_pages == (14, 40) and engine.cache.stats().free_slots == 2
        tokens = rs.tokens_for(70, 150, 77)
        got = engine.run_cuts("long", tokens, list(range(10, 150, 10)), release=False)
        windowed = engine.cache.get("long").pages[0]
        assert windowed[0] < 0 and sum(p >= 0 for p in windowed) <= 5       # only the window's pages are held
        rs.assert_logits_close(got, engine.plain(tokens), F32, "long")


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
