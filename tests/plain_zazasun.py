"""Plain, slow Zazasun decoder: the oracle of the tests of that architecture.

Whole sequences only, no cache, no kernels, one function per mechanism, written from the
architecture's equations token by token where a recurrence is involved.  It shares no code with the
package: it reads tensors by their checkpoint names out of a ``dict`` and sizes and constants out of
the ``config.json`` dictionary.  ``dtype`` is the arithmetic (float64 by default, so that the oracle's
own rounding never shows).

Notation.  W is the width, t a position (from 0 in every sequence), x_t the residual stream.
A layer computes h_t = norm(x_t), s_t = h_t + (h_{t-1} - h_t) * shift (h_{-1} = 0), and
x_t <- x_t + mixer(s)_t + ff(h)_t.
"""

from __future__ import annotations

import math

import torch


def scalar_rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * g with one gain g for the whole row."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * gain


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def shift_mix(h: torch.Tensor, coefficient: torch.Tensor) -> torch.Tensor:
    """h_t + (h_{t-1} - h_t) * c, with zeros before the first token.  h is [T, W]."""
    previous = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (previous - h) * coefficient


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_feed_forward(h, gate, up, down):
    return (gelu_tanh(h @ gate.T) * (h @ up.T)) @ down.T


def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    """window 0 stands for "no window": every earlier key is seen."""
    return j <= i and (not window or i - j < window or j < keep_first)


def differential_attention(h, t, prefix, mixer, eps):
    """Two softmax maps per head over shared values, combined as a1 - lambda * a2."""
    heads, groups, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    mask = mixer.get("mask") or {"size": 0, "keep_first": 0}
    window, keep_first = mask["size"], mask.get("keep_first", 0)
    scale, diff = mixer["scale"], mixer["diff"]
    length = h.shape[0]
    q = (h @ t[prefix + "q"].T).reshape(length, heads, 2, dim)
    k = (h @ t[prefix + "k"].T).reshape(length, groups, 2, dim)
    v = (h @ t[prefix + "v"].T).reshape(length, groups, vdim)
    q = unit_rms(q, eps) * t[prefix + "q.norm"]
    k = unit_rms(k, eps) * t[prefix + "k.norm"]
    lam = (torch.exp((t[prefix + "lq1"] * t[prefix + "lk1"]).sum())
           - torch.exp((t[prefix + "lq2"] * t[prefix + "lk2"]).sum()) + diff)
    out = torch.zeros(length, heads, vdim, dtype=h.dtype)
    for i in range(length):
        keys = [j for j in range(i + 1) if visible(i, j, window, keep_first)]
        for head in range(heads):
            group = head // (heads // groups)
            maps = []
            for m in range(2):
                scores = (k[keys, group, m] @ q[i, head, m]) * scale
                weights = torch.softmax(scores, dim=0)
                maps.append(weights @ v[keys, group])
            o = maps[0] - lam * maps[1]
            out[i, head] = unit_rms(o, eps) * (1.0 - diff)
    return out.reshape(length, heads * vdim) @ t[prefix + "o"].T


def wkv_mixer(h, t, prefix, mixer, eps):
    """Time mixing with a per-channel decay and a bonus for the current token."""
    heads, dim = mixer["heads"], mixer["dim"]
    length = h.shape[0]
    mixes = {name: shift_mix(h, t[prefix + "mu." + name]) for name in "rkvgw"}
    r = (mixes["r"] @ t[prefix + "r"].T).reshape(length, heads, dim)
    k = (mixes["k"] @ t[prefix + "k"].T).reshape(length, heads, dim)
    v = (mixes["v"] @ t[prefix + "v"].T).reshape(length, heads, dim)
    gate = torch.nn.functional.silu(mixes["g"] @ t[prefix + "g"].T)
    raw = torch.tanh(mixes["w"] @ t[prefix + "w1"].T) @ t[prefix + "w2"].T + t[prefix + "w0"]
    w = torch.exp(-torch.exp(raw)).reshape(length, heads, dim)
    u = t[prefix + "u"]
    state = torch.zeros(heads, dim, dim, dtype=h.dtype)      # [head, key channel, value channel]
    out = torch.zeros(length, heads, dim, dtype=h.dtype)
    for step in range(length):
        kv = k[step][:, :, None] * v[step][:, None, :]
        out[step] = torch.einsum("hi,hij->hj", r[step], state + u[:, :, None] * kv)
        state = w[step][:, :, None] * state + kv
    out = unit_rms(out, eps).reshape(length, heads * dim) * t[prefix + "norm"] * gate
    return out @ t[prefix + "o"].T


def hgrn2_mixer(h, t, prefix, mixer, eps):
    """Linear attention whose forget gate f also sets what is written (1 - f)."""
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    length = h.shape[0]
    q = torch.nn.functional.silu(h @ t[prefix + "q"].T).reshape(length, heads, dim)
    v = (h @ t[prefix + "v"].T).reshape(length, heads, vdim)
    lower = t[prefix + "lower"]
    f = lower + (1.0 - lower) * torch.sigmoid(h @ t[prefix + "f"].T + t[prefix + "f.b"])
    f = f.reshape(length, heads, dim)
    state = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    out = torch.zeros(length, heads, vdim, dtype=h.dtype)
    for step in range(length):
        state = f[step][:, :, None] * state + (1.0 - f[step])[:, :, None] * v[step][:, None, :]
        out[step] = torch.einsum("hi,hij->hj", q[step], state)
    out = unit_rms(out, eps) * t[prefix + "norm"]
    return out.reshape(length, heads * vdim) @ t[prefix + "o"].T


MIXERS = {"attention": differential_attention, "wkv": wkv_mixer, "hgrn2": hgrn2_mixer}


def forward(tensors, config, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer if asked)."""
    t = {name: (value.to(dtype) if value.dtype.is_floating_point else value) for name, value in tensors.items()}
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = t["embed"][ids] + t["pos"][: len(tokens)]
    layers = []
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        h = scalar_rms_norm(x, t[prefix + "norm1"], eps)
        shifted = shift_mix(h, t[prefix + "shift"])
        delta = MIXERS[layer["type"]](shifted, t, prefix + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']!r}")
            delta = delta + gated_feed_forward(h, t[prefix + "mlp.gate"], t[prefix + "mlp.up"], t[prefix + "mlp.down"])
        x = x + delta
        layers.append(x)
    logits = scalar_rms_norm(x, t["final.norm"], eps) @ t["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits
