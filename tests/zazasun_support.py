"""Helpers of the Zazasun tests: small configurations of the tests' own, random weights drawn here
(large enough that attention is peaked and the recurrences remember), an engine around the
framework's model, cache manager and step function, and the plain oracle beside it."""

from __future__ import annotations

import math

import torch

import plain_zazasun as plain
from mini_llm_runtime_b200.cache import CacheManager
from mini_llm_runtime_b200.config import config_from_dict
from mini_llm_runtime_b200.engine import ModelRunner, StepEntry
from mini_llm_runtime_b200.models import build_model


def attention(heads, kv_heads, dim, vdim, window, keep_first, diff=0.3, scale=None, ff=0):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
                      "scale": scale if scale is not None else 1.0 / math.sqrt(dim),
                      "mask": {"size": window, "keep_first": keep_first}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def wkv(heads, dim, ff=0):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def hgrn2(heads, dim, vdim, ff=0):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, width, vocab, max_positions=512, eps=1e-5):
    return {"architecture": "Zazasun", "vocab": vocab, "width": width, "max_positions": max_positions,
            "norm": {"eps": eps}, "layers": list(layers)}


# three layers of each kind with a feed-forward on some; every size differs from every other
MIXED = config([hgrn2(3, 16, 24, ff=80), attention(4, 2, 16, 24, window=12, keep_first=3, ff=48),
                wkv(2, 24), attention(2, 2, 24, 16, window=33, keep_first=0, diff=0.7, ff=64)],
               width=96, vocab=131)
# widths and ranks that are no multiple of 8, one kv head, kept positions beyond the window, one head
ODD = config([wkv(3, 40, ff=52), attention(6, 1, 8, 40, window=5, keep_first=7, diff=0.55),
              hgrn2(1, 64, 8, ff=20)], width=68, vocab=77, max_positions=300, eps=3e-6)
# sizes the tensor-core products take (multiples of 64), for bfloat16 and many rows
WIDE = config([attention(4, 2, 64, 64, window=100, keep_first=4, ff=256), wkv(4, 64, ff=256),
               hgrn2(2, 128, 64, ff=128)], width=256, vocab=320, max_positions=1024, eps=1e-6)


def draw_tensors(expected, seed, overrides=None):
    """Random weights by the kind each part declares, stored as bfloat16 (so that the 32-bit and the
    16-bit engine and the oracle all read the same numbers)."""
    generator = torch.Generator().manual_seed(seed)
    tensors = {}
    for name in sorted(expected):
        spec = expected[name]
        shape = tuple(spec.shape)
        if spec.init == "unit":
            value = torch.rand(shape, generator=generator)
        elif spec.init == "norm":
            value = 1.0 + 0.2 * torch.randn(shape, generator=generator)
        elif spec.init == "bias":
            value = 0.5 * torch.randn(shape, generator=generator)
        else:
            fan_in = shape[-1] if len(shape) > 1 else 1
            value = torch.randn(shape, generator=generator) * (1.2 / math.sqrt(fan_in))
        tensors[name] = value
    tensors["embed"] = torch.randn(tensors["embed"].shape, generator=generator)
    tensors["pos"] = 0.5 * torch.randn(tensors["pos"].shape, generator=generator)
    for name, value in (overrides or {}).items():
        tensors[name] = value(tensors[name]) if callable(value) else value
    return {name: value.to(torch.bfloat16) for name, value in tensors.items()}


def long_memory(tensors_expected):
    """Overrides that make the recurrences forget slowly, so that a state lost at a step's border or
    a wrong slot shows hundreds of tokens later."""
    out = {}
    for name in tensors_expected:
        if name.endswith(".mix.w0"):
            out[name] = lambda t: t * 0.2 - 4.0          # decay exp(-exp(-4)) ~ 0.98
        if name.endswith(".mix.lower"):
            out[name] = lambda t: 0.9 + 0.09 * t         # forget gate in (0.9, 1)
    return out


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


class ZEngine:
    def __init__(self, config_dict, dtype, device, *, page_size=16, num_pages=64, max_requests=4, max_tokens=512,
                 seed=0, overrides=None, long=False, max_step_tokens=None):
        self.config_dict = config_dict
        self.dtype = dtype
        self.config = config_from_dict(config_dict)
        self.model = build_model(self.config, dtype)
        expected = self.model.expected_tensors()
        overrides = dict(overrides or {})
        if long:
            overrides = {**long_memory(expected), **overrides}
        self.tensors = draw_tensors(expected, seed, overrides)
        self.model.load(self.tensors, device)
        self.cache = CacheManager(self.model.cache_needs(), page_size=page_size, num_pages=num_pages,
                                  max_requests=max_requests, max_tokens_per_request=max_tokens, dtype=dtype,
                                  device=device, max_step_tokens=max_step_tokens or max_tokens)
        self.runner = ModelRunner(self.model, self.cache)
        self.runner.graph_capture_after = 1

    def plain(self, tokens):
        return plain.forward(self.tensors, self.config_dict, tokens)

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
