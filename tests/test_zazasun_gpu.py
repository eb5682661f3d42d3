"""Zazasun through the framework's model, cache manager, step function and kernels, against the
plain implementation (``plain_zazasun``): whole prompts, token-by-token decoding, portions, mixed
batches, reused pages and slots, window and kept-first edges with a key made to dominate, long
decoding through captured steps, odd sizes, and greedy generation through the scheduler."""

from __future__ import annotations

import pytest
import torch

import plain_zazasun as plain
import zazasun_support as zs
from mini_llm_runtime_b200.engine import ContinuousBatchEngine

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def one_layer(kind):
    layer = {"attention": zs.attention(3, 1, 16, 40, window=9, keep_first=2, ff=0),
             "wkv": zs.wkv(3, 24), "hgrn2": zs.hgrn2(2, 24, 40)}[kind]
    return zs.config([layer], width=72, vocab=90)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["attention", "wkv", "hgrn2"])
def test_each_mixer_alone(kind, dtype):
    engine = zs.ZEngine(one_layer(kind), dtype, DEVICE, seed=11)
    tokens = zs.tokens_for(90, 61, 5)
    zs.assert_logits_close(engine.run_cuts("a", tokens, []), engine.plain(tokens), dtype, kind)


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_alone_and_a_layer_without_one(dtype):
    with_ff = zs.config([zs.hgrn2(2, 16, 16, ff=56)], width=48, vocab=50)
    tokens = zs.tokens_for(50, 20, 3)
    engine = zs.ZEngine(with_ff, dtype, DEVICE, seed=2)
    zs.assert_logits_close(engine.run_cuts("a", tokens, []), engine.plain(tokens), dtype)
    without = zs.config([zs.hgrn2(2, 16, 16)], width=48, vocab=50)
    engine = zs.ZEngine(without, dtype, DEVICE, seed=2)
    zs.assert_logits_close(engine.run_cuts("a", tokens, []), engine.plain(tokens), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["MIXED", "ODD"])
def test_prefill_against_token_by_token(name, dtype):
    config = getattr(zs, name)
    engine = zs.ZEngine(config, dtype, DEVICE, seed=1, long=True)
    tokens = zs.tokens_for(config["vocab"], 75, 8)
    want = engine.plain(tokens)
    zs.assert_logits_close(engine.run_cuts("whole", tokens, []), want, dtype, "whole")
    zs.assert_logits_close(engine.run_cuts("single", tokens, range(1, 75)), want, dtype, "token by token")
    zs.assert_logits_close(engine.run_cuts("tail", tokens, [40] + list(range(41, 75))), want, dtype, "prompt then decode")


@pytest.mark.parametrize("cuts", [[2, 4, 6, 8], [3, 19, 20, 52], [16, 32, 48, 64], [1, 2, 35, 37, 90], [17, 34, 51]])
def test_portions_of_several_sizes(cuts):
    engine = zs.ZEngine(zs.MIXED, torch.float32, DEVICE, seed=4, long=True)
    tokens = zs.tokens_for(131, 100, 9)
    zs.assert_logits_close(engine.run_cuts("a", tokens, cuts), engine.plain(tokens), torch.float32)


def test_float32_logits_do_not_depend_on_the_cut():
    engine = zs.ZEngine(zs.MIXED, torch.float32, DEVICE, seed=4, long=True)
    tokens = zs.tokens_for(131, 90, 10)
    whole = engine.run_cuts("a", tokens, [])
    pieces = engine.run_cuts("b", tokens, [2, 5, 30, 31, 64])
    assert float((whole - pieces).abs().max()) <= 2e-5 * float(whole.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_batches_of_unequal_requests(dtype):
    engine = zs.ZEngine(zs.MIXED, dtype, DEVICE, seed=6, long=True, num_pages=40)
    prompts = {"a": zs.tokens_for(131, 70, 1), "b": zs.tokens_for(131, 41, 2), "c": zs.tokens_for(131, 9, 3),
               "d": zs.tokens_for(131, 100, 4)}
    # portions of some beside single tokens of others; every request at its own place
    plan = [{"a": 30, "b": 1, "d": 2}, {"a": 1, "b": 16, "c": 9, "d": 50}, {"a": 1, "b": 1, "d": 1},
            {"a": 38, "b": 23, "d": 47}]
    got = {name: [] for name in prompts}
    at = {name: 0 for name in prompts}
    for name in prompts:
        engine.cache.create_request(name)
    for step in plan:
        entries = [(name, prompts[name][at[name]:at[name] + count], range(count)) for name, count in step.items()]
        logits = engine.step(entries)
        row = 0
        for name, count in step.items():
            got[name].append(logits[row:row + count])
            row += count
            at[name] += count
    for name, tokens in prompts.items():
        assert at[name] == len(tokens)
        zs.assert_logits_close(torch.cat(got[name]), engine.plain(tokens), dtype, name)


def test_pages_and_slots_are_used_again():
    # 2 slots, 12 pages of 8: a 150-token request only fits because the windowed layers give pages back
    config = zs.config([zs.attention(2, 1, 16, 24, window=20, keep_first=5, ff=32), zs.wkv(2, 16),
                        zs.attention(2, 1, 16, 24, window=20, keep_first=5)], width=64, vocab=70)
    engine = zs.ZEngine(config, torch.float32, DEVICE, seed=3, long=True, page_size=8, num_pages=12, max_requests=2,
                        max_tokens=200, max_step_tokens=32)
    for round_number in range(3):
        names = [f"r{round_number}a", f"r{round_number}b"]
        prompts = [zs.tokens_for(70, 33 + 7 * round_number, 20 + round_number), zs.tokens_for(70, 25, 30 + round_number)]
        outputs = [[], []]
        for name in names:
            engine.cache.create_request(name)
        for start in range(0, 60, 6):
            entries = [(name, prompt[start:start + 6], range(len(prompt[start:start + 6])))
                       for name, prompt in zip(names, prompts) if start < len(prompt)]
            if not entries:
                break
            logits = engine.step(entries)
            row = 0
            for index, (name, prompt) in enumerate(zip(names, prompts)):
                count = len(prompt[start:start + 6])
                if start < len(prompt):
                    outputs[index].append(logits[row:row + count])
                    row += count
        for index, (name, prompt) in enumerate(zip(names, prompts)):
            zs.assert_logits_close(torch.cat(outputs[index]), engine.plain(prompt), torch.float32, name)
            engine.cache.release(name)
        engine.cache.check_consistency()
    assert engine.cache.stats().free_pages == (12,)
    # a long request alone: its pages beyond the window come back while it runs, the first page stays
    tokens = zs.tokens_for(70, 150, 77)
    got = engine.run_cuts("long", tokens, list(range(10, 150, 10)), release=False)
    held = engine.cache.get("long").pages[0]
    assert held[0] >= 0 and held[1] < 0 and sum(p >= 0 for p in held) <= 6
    zs.assert_logits_close(got, engine.plain(tokens), torch.float32, "long")


# ---------------------------------------------------------------- a key made to dominate
def dominant_key_case(window, keep_first, length, query, key, seed):
    """A one-layer attention model whose weights let one chosen key dominate one chosen query: token
    ids are positions' own (vocabulary = length); the query's token embeds as a large vector a, the
    key's token as a rolled by one channel, and the key projection is the query projection rolled the
    same way, so that k(key) equals q(query) of the first head while no other key (the query's own
    included) points that way.  Everything else is small; shift coefficients are zero."""
    config = zs.config([zs.attention(2, 1, 8, 12, window=window, keep_first=keep_first, diff=0.2, scale=2.0)],
                       width=40, vocab=length, max_positions=length)
    generator = torch.Generator().manual_seed(seed)

    def embed(table):
        table = 0.3 * torch.randn(table.shape, generator=generator)
        special = 3.0 * torch.randn(table.shape[1], generator=generator)
        table[key] = torch.roll(special, 1)
        table[query] = special
        return table

    overrides = {"embed": embed, "pos": lambda t: torch.zeros_like(t), "l0.shift": lambda t: torch.zeros_like(t)}
    return config, overrides


@pytest.mark.parametrize("how", ["prompt", "decoded", "portions"])
@pytest.mark.parametrize("window,keep_first,query,key", [
    (10, 3, 40, 31),     # just inside the window
    (10, 3, 40, 30),     # just outside
    (10, 3, 290, 2),     # far back, among the kept first positions
    (10, 3, 290, 3),     # the first position that is not kept
    (16, 0, 47, 32),     # a window's edge on a page's border, nothing kept
    (16, 16, 100, 15),   # the last kept position, the last place of a page
])
def test_window_and_kept_first_edges_with_a_dominant_key(window, keep_first, query, key, how):
    length = 300
    config, overrides = dominant_key_case(window, keep_first, length, query, key, seed=query + key)
    engine = zs.ZEngine(config, torch.float32, DEVICE, seed=5, overrides=overrides, num_pages=24, max_tokens=320)
    engine.tensors["l0.mix.k"] = torch.roll(engine.tensors["l0.mix.q"][:16], 1, dims=1).contiguous()
    engine.model.load(engine.tensors, DEVICE)
    tokens = list(range(length))
    want = engine.plain(tokens)
    cuts = {"prompt": [], "decoded": [20] + list(range(21, length)), "portions": [7, query - 1, query, query + 2]}[how]
    got = engine.run_cuts("a", tokens, cuts)
    zs.assert_logits_close(got[query:query + 1], want[query:query + 1], torch.float32, f"query {query}")
    zs.assert_logits_close(got, want, torch.float32)
    # the case tells: with the edge moved by one position the oracle's answer at the query changes visibly
    moved = dict(config)
    layer = {**config["layers"][0], "mixer": {**config["layers"][0]["mixer"]}}
    inside = plain.visible(query, key, window, keep_first)
    if key <= keep_first and query - key > window:       # a kept-first edge
        layer["mixer"]["mask"] = {"size": window, "keep_first": keep_first + (-1 if inside else 1)}
    else:
        layer["mixer"]["mask"] = {"size": window + (-1 if inside else 1), "keep_first": keep_first}
    moved["layers"] = [layer]
    other = plain.forward(engine.tensors, moved, tokens)
    assert float((other[query] - want[query]).abs().max()) > 1e-2 * float(want[query].abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_through_captured_steps(dtype):
    engine = zs.ZEngine(zs.MIXED, dtype, DEVICE, seed=12, long=True, num_pages=64)
    tokens = zs.tokens_for(131, 260, 13)
    want = engine.plain(tokens)
    got = engine.run_cuts("a", tokens, [30] + list(range(31, 260)))
    assert engine.runner.graph_replays > 100
    zs.assert_logits_close(got, want, dtype)
    # two requests decoding side by side through the captured step of two
    other = zs.tokens_for(131, 60, 14)
    engine.cache.create_request("x")
    engine.cache.create_request("y")
    first = engine.step([("x", tokens[:20], range(20)), ("y", other[:10], range(10))])
    rows = {"x": [first[:20]], "y": [first[20:]]}
    for i in range(40):
        logits = engine.step([("x", tokens[20 + i:21 + i], [0]), ("y", other[10 + i:11 + i], [0])])
        rows["x"].append(logits[:1])
        rows["y"].append(logits[1:])
    zs.assert_logits_close(torch.cat(rows["x"]), want[:60], dtype, "x")
    zs.assert_logits_close(torch.cat(rows["y"]), engine.plain(other[:50]), dtype, "y")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_the_tensor_core_products_take(dtype):
    engine = zs.ZEngine(zs.WIDE, dtype, DEVICE, seed=21, long=True, num_pages=80, max_tokens=1024)
    tokens = zs.tokens_for(320, 420, 22)
    want = engine.plain(tokens)
    zs.assert_logits_close(engine.run_cuts("a", tokens, [300, 301, 302, 350]), want, dtype)


def test_greedy_generation_through_the_scheduler():
    engine_parts = zs.ZEngine(zs.MIXED, torch.float32, DEVICE, seed=31, long=True)
    engine = ContinuousBatchEngine.from_model(engine_parts.model, block_size=8, total_blocks=96, max_running_requests=3,
                                              max_batch_tokens=24, max_model_len=160)
    prompts = [zs.tokens_for(131, length, 40 + i) for i, length in enumerate([5, 37, 18, 50, 2])]
    generated = engine.generate(prompts, max_new_tokens=12)
    for prompt, got in zip(prompts, generated):
        sequence = list(prompt)
        for _ in range(12):
            sequence.append(int(torch.argmax(engine_parts.plain(sequence)[-1])))
        assert got == sequence[len(prompt):]


@pytest.mark.parametrize("rows", [1, 8, 40, 130, 700])
@pytest.mark.parametrize("inner,width", [(256, 128), (1216, 896)])
def test_gated_product_with_the_gelu_epilogue(rows, inner, width):
    """gelu_tanh(x Wg^T) * (x Wu^T) from the products' own epilogues (few rows, many rows) against
    the formula, on weights interleaved in blocks of 64."""
    from mini_llm_runtime_b200 import ops

    generator = torch.Generator().manual_seed(rows + inner)
    x = torch.randn(rows, width, generator=generator).to(torch.bfloat16)
    gate = (torch.randn(inner, width, generator=generator) / width ** 0.5 * 2).to(torch.bfloat16)
    up = (torch.randn(inner, width, generator=generator) / width ** 0.5).to(torch.bfloat16)
    stacked = torch.cat([gate.view(-1, 64, width), up.view(-1, 64, width)], dim=1).reshape(2 * inner, width)
    got = ops.current().linear_gated(x.to(DEVICE), stacked.to(DEVICE).contiguous(), 64, "gelu_tanh")
    want = plain.gelu_tanh(x.double() @ gate.double().T) * (x.double() @ up.double().T)
    error = (got.double().cpu() - want).abs().max() / want.abs().max()
    assert float(error) < 1e-2


def test_command_line_and_replay_program_with_a_model_folder(tmp_path):
    """``make-random`` writes a Zazasun folder from a config.json, ``generate`` reproduces the plain
    implementation's greedy tokens from it, and the replay program writes the logits of the wanted
    places step by step, with pages and slots given back in between."""
    import json
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

    (tmp_path / "config.json").write_text(json.dumps(zs.ODD))
    folder = tmp_path / "model"
    cli("-m", "mini_llm_runtime_b200", "make-random", "--config", str(tmp_path / "config.json"), "--seed", "4",
        "--out", str(folder))
    tensors = read_checkpoint(folder)
    prompt = zs.tokens_for(77, 11, 6)
    sequence = list(prompt)
    for _ in range(5):
        sequence.append(int(torch.argmax(plain.forward(tensors, zs.ODD, sequence)[-1])))
    record = json.loads(cli("-m", "mini_llm_runtime_b200", "generate", "--model", str(folder), "--dtype", "float32",
                            "--max-model-len", "64", "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "5"
                            ).splitlines()[-1])
    assert record["generated_ids"] == sequence[len(prompt):]

    other = zs.tokens_for(77, 30, 7)
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": prompt[:4], "want": [0, 3]}], "end": []},
             {"step": 1, "entries": [{"id": "p", "tokens": prompt[4:], "want": [6]},
                                     {"id": "o", "tokens": other, "want": [29]}], "end": ["p"]},
             {"step": 2, "entries": [], "end": ["o"]}]
    out = cli(os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out",
              str(tmp_path / "logits"), "--max-tokens", "64", stdin="\n".join(json.dumps(s) for s in steps) + "\n")
    assert [line for line in out.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    first = torch.from_numpy(np.fromfile(tmp_path / "logits" / "0.f32", dtype="<f4").reshape(2, 77))
    second = torch.from_numpy(np.fromfile(tmp_path / "logits" / "1.f32", dtype="<f4").reshape(2, 77))
    want = plain.forward(tensors, zs.ODD, prompt)
    zs.assert_logits_close(torch.cat([first, second[:1]]), want[[0, 3, 10]], torch.float32)
    zs.assert_logits_close(second[1:], plain.forward(tensors, zs.ODD, other)[29:], torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
def test_state_heads_larger_than_one_block_of_threads_holds(dtype):
    """A 256 x 256 state per head, and value heads whose size is no multiple of 32: the recurrence
    spreads the value channels over several blocks (in prompt steps always, in decode steps when a
    head does not fit one block), the last part being short."""
    config = zs.config([zs.wkv(1, 256), zs.hgrn2(1, 40, 200, ff=32)], width=64, vocab=60)
    engine = zs.ZEngine(config, dtype, DEVICE, seed=8, long=True)
    tokens = zs.tokens_for(60, 90, 4)
    want = engine.plain(tokens)
    zs.assert_logits_close(engine.run_cuts("a", tokens, []), want, dtype, "whole")
    zs.assert_logits_close(engine.run_cuts("b", tokens, [70, 71, 72, 80]), want, dtype, "portions and single tokens")
