"""Zazasun's host side without a GPU: configuration and registry, weight checks, the cache manager's
kept pages and several states per entry, and the whole engine (step function, scheduler, replay
program's loop) on the stand-in kernels against the plain implementation."""

from __future__ import annotations

import json

import pytest
import torch

import zazasun_support as zs
from fake_ops import FakeOps
from mini_llm_runtime_b200 import ops
from mini_llm_runtime_b200.cache import CacheManager
from mini_llm_runtime_b200.config import ZazasunConfig, config_from_dict, load_config
from mini_llm_runtime_b200.engine import ContinuousBatchEngine
from mini_llm_runtime_b200.models import build_model, load_model, write_random_model_dir
from mini_llm_runtime_b200.parts import KVCacheNeed, StateNeed
from mini_llm_runtime_b200.weights.loader import WeightError


def test_config_round_trip_and_registry(tmp_path):
    config = config_from_dict(zs.MIXED)
    assert isinstance(config, ZazasunConfig) and config.vocab_size == 131 and len(config.layers) == 4
    assert config_from_dict(config.to_dict()) == config
    assert config.to_dict()["layers"][2]["mlp"] is None
    folder = write_random_model_dir(tmp_path / "model", config, seed=3)
    entry, loaded = load_config(folder)
    assert entry.name == "Zazasun" and loaded == config
    stored = json.loads((folder / "config.json").read_text())
    assert stored["architecture"] == "Zazasun" and stored["layers"][1]["mixer"]["mask"] == {"size": 12, "keep_first": 3}


@pytest.mark.parametrize("damage,message", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "kind"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "layer"),
])
def test_config_errors(damage, message):
    data = json.loads(json.dumps(zs.MIXED))
    damage(data)
    with pytest.raises((KeyError, ValueError), match=message):
        config_from_dict(data)


def test_expected_tensors_and_a_bottleneck_width_taken_from_the_checkpoint():
    model = build_model(config_from_dict(zs.ODD), torch.float32)
    expected = model.expected_tensors()
    assert expected["l0.norm1"].shape == () and expected["final.norm"].shape == ()
    assert expected["l1.mix.q"].shape == (2 * 6 * 8, 68) and expected["l1.mix.k"].shape == (2 * 8, 68)
    assert expected["l1.mix.v"].shape == (40, 68) and expected["l2.mix.norm"].shape == (8,)
    assert "l1.mlp.gate" not in expected and expected["l0.mlp.down"].shape == (68, 52)
    tensors = zs.draw_tensors(expected, 1)
    with ops.use(FakeOps()):
        # another bottleneck width than the default is accepted when both matrices agree ...
        tensors["l0.mix.w1"] = torch.zeros(5, 68, dtype=torch.bfloat16)
        tensors["l0.mix.w2"] = torch.zeros(120, 5, dtype=torch.bfloat16)
        model.load(tensors, "cpu")
        # ... and refused when they do not, or when a fixed size is off
        tensors["l0.mix.w2"] = torch.zeros(120, 6, dtype=torch.bfloat16)
        with pytest.raises(ValueError, match="bottleneck"):
            build_model(config_from_dict(zs.ODD), torch.float32).load(tensors, "cpu")
        tensors["l0.mix.w2"] = torch.zeros(121, 5, dtype=torch.bfloat16)
        with pytest.raises(WeightError):
            build_model(config_from_dict(zs.ODD), torch.float32).load(tensors, "cpu")


def test_cache_needs_of_every_layer_kind():
    model = build_model(config_from_dict(zs.MIXED), torch.float32)
    needs = model.cache_needs()
    assert needs[0] == (StateNeed((3, 16, 24), torch.float32, "state"), StateNeed((96,), torch.float32, "shift"))
    assert needs[1] == (KVCacheNeed(2, 32, 12, value_dim=24, keep_first=3), StateNeed((96,), torch.float32, "shift"))
    assert needs[2] == (StateNeed((2, 24, 24), torch.float32, "state"),
                        StateNeed((96,), torch.float32, "previous_input"), StateNeed((96,), torch.float32, "shift"))
    assert needs[3][0] == KVCacheNeed(2, 48, 33, value_dim=16, keep_first=0)


def test_kept_pages_stay_while_the_window_moves_on():
    need = (KVCacheNeed(1, 8, window=10, value_dim=4, keep_first=5), StateNeed((3,), torch.float32, "shift"))
    m = CacheManager([need], page_size=4, num_pages=12, max_requests=2, max_tokens_per_request=200,
                     dtype=torch.float32, device="cpu", max_step_tokens=8)
    assert m.groups[0].kept_pages == 2 and m.groups[0].value.shape[-1] == 4 and m.groups[0].key.shape[-1] == 8
    request = m.create_request("a")
    for _ in range(12):
        m.begin_step([("a", 8)])
        m.commit_step()
        m.check_consistency()
    pages = request.pages[0]
    # 96 tokens: pages 0 and 1 hold the kept positions; the next query (96) sees keys 87.. = page 21 on
    assert pages[0] >= 0 and pages[1] >= 0 and all(p < 0 for p in pages[2:21]) and all(p >= 0 for p in pages[21:24])
    assert m.pages_for_lifetime(m.groups[0], 1000) == -(-(10 - 1 + 8) // 4) + 1 + 2
    m.release("a")
    assert m.stats().free_pages == (12,)


def test_every_state_of_an_entry_is_zeroed_on_reuse_and_restored_on_abort():
    need = (StateNeed((2,), torch.float32, "state"), StateNeed((3,), torch.float32, "shift"))
    m = CacheManager([need], page_size=4, num_pages=1, max_requests=1, max_tokens_per_request=16,
                     dtype=torch.float32, device="cpu")
    a = m.create_request("a")
    assert set(m.states[0]) == {"state", "shift"} and m.state[0] is m.states[0]["state"]
    m.begin_step([("a", 1)])
    m.states[0]["shift"][a.slot] += 7
    m.states[0]["state"][a.slot] += 5
    m.abort_step()
    assert float(m.states[0]["shift"].abs().sum()) == 0 and float(m.state[0].abs().sum()) == 0
    m.begin_step([("a", 1)])
    m.states[0]["shift"][a.slot] += 7
    m.commit_step()
    m.release("a")
    assert float(m.states[0]["shift"][m.create_request("b").slot].abs().sum()) == 0
    with pytest.raises(ValueError, match="twice"):
        CacheManager([(StateNeed((1,)), StateNeed((2,)))], page_size=4, num_pages=1, max_requests=1,
                     max_tokens_per_request=4, dtype=torch.float32, device="cpu")


@pytest.mark.parametrize("name", ["MIXED", "ODD"])
def test_engine_on_the_stand_in_kernels(name):
    config = getattr(zs, name)
    with ops.use(FakeOps()):
        engine = zs.ZEngine(config, torch.float32, "cpu", seed=2, long=True, page_size=8, num_pages=24, max_tokens=96)
        tokens = zs.tokens_for(config["vocab"], 45, 1)
        other = zs.tokens_for(config["vocab"], 30, 2)
        want, want_other = engine.plain(tokens), engine.plain(other)
        zs.assert_logits_close(engine.run_cuts("a", tokens, [2, 17, 18, 40]), want, torch.float32)
        engine.cache.create_request("x")
        engine.cache.create_request("y")
        first = engine.step([("x", tokens[:20], range(20)), ("y", other[:1], [0])])
        second = engine.step([("y", other[1:30], range(29)), ("x", tokens[20:21], [0])])
        third = engine.step([("x", tokens[21:45], range(24))])
        zs.assert_logits_close(torch.cat([first[:20], second[29:], third]), want, torch.float32, "x")
        zs.assert_logits_close(torch.cat([first[20:], second[:29]]), want_other, torch.float32, "y")


def test_greedy_generation_through_the_scheduler_on_the_stand_in_kernels():
    with ops.use(FakeOps()):
        parts = zs.ZEngine(zs.MIXED, torch.float32, "cpu", seed=31, long=True)
        engine = ContinuousBatchEngine.from_model(parts.model, block_size=8, total_blocks=48, max_running_requests=2,
                                                  max_batch_tokens=16, max_model_len=80)
        prompts = [zs.tokens_for(131, length, 40 + i) for i, length in enumerate([5, 27, 2])]
        generated = engine.generate(prompts, max_new_tokens=6)
        for prompt, got in zip(prompts, generated):
            sequence = list(prompt)
            for _ in range(6):
                sequence.append(int(torch.argmax(parts.plain(sequence)[-1])))
            assert got == sequence[len(prompt):]
        assert engine.manager.stats().live_requests == 0 and engine.manager.stats().free_slots == 2


def test_a_model_folder_loads_through_the_registry(tmp_path):
    config = config_from_dict(zs.ODD)
    folder = write_random_model_dir(tmp_path / "m", config, seed=9)
    with ops.use(FakeOps()):
        loaded, model = load_model(folder, "float32", "cpu", arena=False)
    assert loaded == config and model.spec.architecture == "Zazasun" and len(model.blocks) == 3
