"""Plain, slow Rozesun decoder: the oracle of the tests of that architecture.

Whole sequences only, no cache, no kernels, one function per mechanism.  It shares no code with the
package: it reads tensors by their checkpoint names out of a ``dict`` and sizes and constants out of
the ``config.json`` dictionary.  ``dtype`` is the arithmetic (float64 by default, so that the oracle's
own rounding never shows).

Notation.  T tokens at positions 0..T-1, stream x [T, W].  A layer is
x <- x + LN1b(mixer(LN1(x))), then x <- x + LN2b(ff(LN2(x))); a run of layers may be passed through
several times in a row with the same weights, a learned vector being added to x before every pass.
"""

from __future__ import annotations

import math

import torch


def layer_norm(x, weight, bias, eps):
    mean = x.mean(dim=-1, keepdim=True)
    centred = x - mean
    variance = (centred * centred).mean(dim=-1, keepdim=True)
    return centred / torch.sqrt(variance + eps) * weight + bias


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def rotate(vector, positions, base, dims, interleaved):
    """Turn the first ``dims`` numbers of the last axis by the positions' angles.  vector is
    [T, ..., n]; pairs are (i, i + dims/2) or, interleaved, (2i, 2i + 1); pair i turns by
    position * base^(-2i/dims)."""
    out = vector.clone()
    half = dims // 2
    for i in range(half):
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        angle = positions.to(vector.dtype) * (base ** (-2.0 * i / dims))
        shape = (-1,) + (1,) * (vector.dim() - 2)
        cos, sin = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
        u, v = vector[..., a], vector[..., b]
        out[..., a] = u * cos - v * sin
        out[..., b] = v * cos + u * sin
    return out


def sees(i: int, j: int, window: int) -> bool:
    """window 0: causal without a window."""
    return j <= i and (not window or i - j < window)


def latent_attention(h, t, prefix, mixer, eps, *, interleaved, sink, gate_per_head):
    """Attention whose queries, keys and values come out of low-rank latents.  Keys are, per head,
    an unrotated part made from the latent and one rotated part that all heads share."""
    heads, dim, rot_dim, vdim = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"]
    rank = mixer["kv_rank"]
    base, dims = mixer["rot"]["base"], mixer["rot"]["dims"]
    window = (mixer.get("mask") or {}).get("size", 0)
    length = h.shape[0]
    positions = torch.arange(length)
    query_latent = rms_norm(h @ t[prefix + "dq"].T, t[prefix + "dq.norm"], eps)
    q = (query_latent @ t[prefix + "uq"].T).reshape(length, heads, dim + rot_dim)
    q_plain, q_turned = q[..., :dim], rotate(q[..., dim:], positions, base, dims, interleaved)
    down = h @ t[prefix + "dkv"].T
    latent = rms_norm(down[:, :rank], t[prefix + "dkv.norm"], eps)
    k_turned = rotate(down[:, rank:], positions, base, dims, interleaved)          # [T, rot_dim], one for all heads
    k_plain = (latent @ t[prefix + "uk"].T).reshape(length, heads, dim)
    value = (latent @ t[prefix + "uv"].T).reshape(length, heads, vdim)
    out = torch.zeros(length, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        scores = (q_plain[:, head] @ k_plain[:, head].T + q_turned[:, head] @ k_turned.T) * mixer["scale"]
        for i in range(length):
            keys = [j for j in range(length) if sees(i, j, window)]
            s = scores[i, keys]
            top = s.max()
            if sink:
                top = torch.maximum(top, t[prefix + "sink"][head])
            weights = torch.exp(s - top)
            total = weights.sum()
            if sink:
                total = total + torch.exp(t[prefix + "sink"][head] - top)
            out[i, head] = (weights / total) @ value[keys, head]
    gate = torch.sigmoid(h @ t[prefix + "g"].T)
    if gate_per_head:
        out = out * gate[:, :, None]
        out = out.reshape(length, heads * vdim)
    else:
        out = out.reshape(length, heads * vdim) * gate
    return out @ t[prefix + "o"].T


def clamped_feed_forward(h, t, prefix, limit):
    g = torch.clamp(h @ t[prefix + "gate"].T, max=limit)
    u = torch.clamp(h @ t[prefix + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ t[prefix + "down"].T


MIXERS = {
    "latent_attention": dict(interleaved=False, sink=False, gate_per_head=False),
    "latent_attention_2": dict(interleaved=True, sink=True, gate_per_head=True),
}


def layer(x, t, index, entry, eps):
    p = f"l{index}."
    h = layer_norm(x, t[p + "norm1"], t[p + "norm1.b"], eps)
    mixer = dict(entry["mixer"])
    if entry["type"] == "latent_attention":
        mixer.pop("mask", None)                       # this kind has no window
    mixed = latent_attention(h, t, p + "mix.", mixer, eps, **MIXERS[entry["type"]])
    x = x + layer_norm(mixed, t[p + "norm1b"], t[p + "norm1b.b"], eps)
    if entry.get("mlp") is not None:
        h = layer_norm(x, t[p + "norm2"], t[p + "norm2.b"], eps)
        passed = clamped_feed_forward(h, t, p + "mlp.", entry["mlp"]["limit"])
        x = x + layer_norm(passed, t[p + "norm2b"], t[p + "norm2b.b"], eps)
    return x


def run_order(config):
    """(layer index, pass number or None) in the order the layers run; the pass number is given at
    the first layer of a pass."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["times"] < 1 or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(count)]
    order = [(i, None) for i in range(loop["start"])]
    for number in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, number if i == loop["start"] else None))
    order += [(i, None) for i in range(loop["stop"], count)]
    return order


def forward(config, tensors, tokens, dtype=torch.float64, streams=None):
    """Logits [T, vocab] of one sequence.  ``streams`` (a list) receives x after every layer run."""
    t = {name: value.to(dtype) if value.is_floating_point() else value for name, value in tensors.items()}
    eps = config["norm"]["eps"]
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for index, number in run_order(config):
        if number is not None:
            x = x + t["loop.step"][number]
        x = layer(x, t, index, config["layers"][index], eps)
        if streams is not None:
            streams.append(x.clone())
    x = layer_norm(x, t["final.norm"], t["final.norm.b"], eps)
    return (x @ t["embed"].T) * config["logit_scale"]
