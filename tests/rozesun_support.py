"""Helpers of the Rozesun tests: small configurations of the tests' own, random weights drawn here
(large enough that attention is peaked), an engine around the framework's model, cache manager and
step function on any device, and the plain oracle beside it."""

from __future__ import annotations

import math

import torch

import plain_rozesun as plain
from mini_llm_runtime_b200.cache import CacheManager
from mini_llm_runtime_b200.config import config_from_dict
from mini_llm_runtime_b200.engine import ModelRunner, StepEntry
from mini_llm_runtime_b200.models import build_model


def _mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, base, scale, dims):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "rot": {"base": base, "dims": rot_dim if dims is None else dims},
            "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}


def _mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit} if ff else None


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, *, base=10000.0, scale=None, dims=None, ff=0, limit=2.0):
    """All earlier keys, rotate-half pairs, plain softmax, a gate per channel."""
    return {"type": "latent_attention", "mixer": _mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, base, scale, dims),
            "mlp": _mlp(ff, limit)}


def latent2(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, *, base=10000.0, scale=None, dims=None, ff=0, limit=2.0):
    """A sliding window, interleaved pairs, a sink per head, a gate per head."""
    mixer = _mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, base, scale, dims)
    mixer["mask"] = {"size": window}
    return {"type": "latent_attention_2", "mixer": mixer, "mlp": _mlp(ff, limit)}


def config(layers, width, vocab, *, loop=None, eps=1e-5, logit_scale=1.0):
    out = {"architecture": "Rozesun", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "logit_scale": logit_scale, "layers": list(layers)}
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# every size differs from every other; the middle two layers run twice; one layer has no feed-forward
MIXED = config([latent2(3, 16, 8, 24, 40, 48, window=12, ff=80, limit=0.8),
                latent(4, 8, 16, 16, 32, 24, base=500.0, ff=48, limit=1.1),
                latent(2, 24, 8, 8, 24, 56),
                latent2(2, 8, 4, 16, 16, 8, window=33, base=77.0, ff=64, limit=0.5)],
               width=96, vocab=131, loop=(1, 3, 2), logit_scale=0.7)
# sizes that are no multiple of 8, one head, a window shorter than a page, rotation of a part of the turned
# entries, a loop of a single pass over the first layer, one layer
ODD = config([latent2(1, 10, 6, 7, 20, 12, window=5, dims=4, ff=52, limit=0.9)],
             width=68, vocab=77, loop=(0, 1, 1), eps=3e-6, logit_scale=1.9)
# no loop at all, equal sizes everywhere (values a given model may happen to make equal)
PLAIN = config([latent(2, 16, 16, 16, 16, 16, ff=16, limit=1.0), latent2(2, 16, 16, 16, 16, 16, window=16, ff=16, limit=1.0)],
               width=32, vocab=40)
# sizes the tensor-core products take (multiples of 64), for bfloat16 and many rows; a loop of three
WIDE = config([latent(4, 64, 32, 64, 128, 192, ff=384, limit=1.2), latent2(2, 64, 64, 128, 192, 128, window=100, ff=384, limit=1.2)],
              width=320, vocab=520, loop=(0, 2, 3), eps=1e-6, logit_scale=1.5)


def draw_tensors(expected, seed, overrides=None):
    """Random weights by the kind each part declares, stored as bfloat16 (so that the 32-bit and the
    16-bit engine and the oracle all read the same numbers)."""
    generator = torch.Generator().manual_seed(seed)
    tensors = {}
    for name in sorted(expected):
        spec = expected[name]
        shape = tuple(spec.shape)
        if spec.init == "norm":
            value = 1.0 + 0.2 * torch.randn(shape, generator=generator)
        elif spec.init == "bias":
            value = 0.5 * torch.randn(shape, generator=generator)
        else:
            fan_in = shape[-1] if len(shape) > 1 else 1
            value = torch.randn(shape, generator=generator) * (1.2 / math.sqrt(fan_in))
        tensors[name] = value
    tensors["embed"] = torch.randn(tensors["embed"].shape, generator=generator)
    for name, value in (overrides or {}).items():
        tensors[name] = value(tensors[name]) if callable(value) else value
    return {name: value.to(torch.bfloat16) for name, value in tensors.items()}


def tokens_for(vocab, length, seed):
    return torch.randint(0, vocab, (length,), generator=torch.Generator().manual_seed(seed)).tolist()


def assert_logits_close(got, want, dtype, what=""):
    """Difference of the rows with their mean taken off, root mean square over the vocabulary,
    relative to the logits' own spread: 2e-5 in 32-bit (order of additions only), 3e-2 in bfloat16."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} against {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    spread = float(want.std())
    delta = got - want
    delta = delta - delta.mean(dim=-1, keepdim=True)
    error = delta.pow(2).mean(dim=-1).sqrt() / spread
    limit = 2e-5 if dtype == torch.float32 else 3e-2
    worst = int(error.argmax())
    assert float(error.max()) <= limit, f"{what}: row {worst} is off by {float(error.max()):.3e} (allowed {limit:.0e})"


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

    def reload(self):
        self.model.load(self.tensors, self.device)

    def plain(self, tokens, config_dict=None):
        return plain.forward(config_dict or self.config_dict, self.tensors, tokens)

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


def dominant_key_case(kind, window, length, query, key, seed):
    """A one-layer model whose weights let one chosen key dominate one chosen query.  Token ids are the
    positions' own (vocabulary = length).  Both latents are the first ``rank`` channels of the normalised
    input (identity projections, unit norm weights); the key matrix of every head is the identity and
    the query matrix a strong roll by one channel, so that score(i, j) ~ roll(c_i) . c_j.  The key's
    token embeds as the query's with those channels rolled, hence c_key = roll(c_query): that one key
    collects nearly all the weight of that one query whenever it is visible, and no other key (the
    query's own included) does.  The turned parts are small."""
    rank, rot, width = 12, 4, 40
    layer = (latent2(2, rank, rot, 10, rank, rank, window, scale=1.0) if kind == "latent_attention_2"
             else latent(2, rank, rot, 10, rank, rank, scale=1.0))
    cfg = config([layer], width=width, vocab=length, logit_scale=1.0)
    generator = torch.Generator().manual_seed(seed)
    eye = torch.eye(rank)

    def embed(table):
        table = torch.randn(table.shape, generator=generator)
        table[key, :rank] = torch.roll(table[query, :rank], 1)
        table[key, rank:] = table[query, rank:]
        return table

    def down(rows):      # [rows, width]: the identity on the first channels
        return torch.cat([torch.eye(rows), torch.zeros(rows, width - rows)], dim=1)

    def query_up(matrix):
        per_head = torch.cat([2.5 * torch.roll(eye, 1, dims=0), 0.05 * torch.randn(rot, rank, generator=generator)])
        return torch.cat([per_head, per_head])

    overrides = {
        "embed": embed,
        "l0.norm1": lambda t: torch.ones_like(t), "l0.norm1.b": lambda t: torch.zeros_like(t),
        "l0.mix.dq": lambda t: down(rank), "l0.mix.dq.norm": lambda t: torch.ones_like(t),
        "l0.mix.dkv": lambda t: torch.cat([down(rank), 0.05 * torch.randn(rot, width, generator=generator)]),
        "l0.mix.dkv.norm": lambda t: torch.ones_like(t),
        "l0.mix.uk": lambda t: torch.cat([eye, eye]), "l0.mix.uq": query_up,
    }
    return cfg, overrides


def random_config(seed):
    """A configuration drawn from a seed: layer kinds in any order, sizes of every parity, a loop
    anywhere (or none), layers with and without a feed-forward."""
    import random

    rng = random.Random(seed)
    count = rng.randint(2, 5)
    layers = []
    for _ in range(count):
        heads, dim, rot_dim = rng.randint(1, 9), rng.choice([4, 6, 8, 10, 16, 24]), rng.choice([2, 4, 8, 12, 16])
        vdim, kv_rank, q_rank = rng.choice([3, 8, 12, 16, 20]), rng.choice([8, 12, 16, 24, 40, 72]), rng.choice([5, 8, 16, 28])
        ff = rng.choice([0, 24, 40, 64])
        options = dict(base=rng.choice([30.0, 1000.0, 50000.0]), scale=rng.choice([None, 0.2, 0.4]),
                       dims=rng.choice([None, rot_dim, max(2, rot_dim - 2)]), ff=ff, limit=rng.choice([0.5, 1.0, 3.0]))
        if rng.random() < 0.5:
            layers.append(latent2(heads, dim, rot_dim, vdim, kv_rank, q_rank, rng.choice([1, 3, 16, 17, 40, 200]), **options))
        else:
            layers.append(latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, **options))
    loop = None
    if rng.random() < 0.7:
        start = rng.randint(0, count - 1)
        loop = (start, rng.randint(start + 1, count), rng.randint(1, 3))
    return config(layers, width=rng.choice([24, 36, 64, 72]), vocab=rng.choice([31, 64, 100]), loop=loop,
                  eps=rng.choice([1e-6, 1e-5, 1e-3]), logit_scale=rng.choice([0.5, 1.0, 2.5]))
