"""Mixers that carry a matrix-valued state per head instead of a key/value cache.

Both keep, per request and head, a state S [dim, vdim] of 32-bit floats that starts at zero and is
advanced token by token; what enters the recurrence beside the projections (decays, gates, norms)
is 32-bit.  Projections leave as 32-bit rows so that nothing is rounded on the way into the
recurrence; the mixer's output projection leaves 32-bit rows for a 32-bit residual stream.

``wkv``    time mixing with a data-dependent per-channel decay and a bonus for the current token:
           every projection reads its own blend of the input with the previous token's input
           (coefficients ``mu.*``); w_t = exp(-exp(W2 tanh(W1 x_w) + w0));
           o_t = (S + diag(u) k_t v_t^T)^T r_t;  S <- diag(w_t) S + k_t v_t^T;
           out = Wo (o / rms(o) * norm * silu(Wg x_g)).
``hgrn2``  gated linear attention whose forget gate also sets what is written:
           f_t = l + (1 - l) sigmoid(Wf x + b);  S <- diag(f_t) S + (1 - f_t) v_t^T;
           o_t = S^T silu(Wq x);  out = Wo (o / rms(o) * norm).
"""

from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import Mixer, StateNeed, TensorSpec, build_part, register_part


def _float(tensor, device):
    return tensor.to(device=device, dtype=torch.float32).contiguous()


class WKVMixer(Mixer):
    graph_safe = True
    wants_float_input = True       # its own blends are taken of 32-bit rows

    BLENDS = ("r", "k", "v", "g", "w")

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.heads = int(a["heads"])
        self.dim = int(a["dim"])
        self.eps = float(a["eps"])
        self.inner = self.heads * self.dim
        # the decay's bottleneck width is whatever the checkpoint's w1/w2 have; random weights use this
        self.default_rank = int(a.get("decay_rank") or max(16, self.hidden_size // 16))
        # the blends with the previous token's input: a token shift with five coefficient vectors
        self.blend = build_part("shift", PartSpec("token_shift", {
            "hidden_size": self.hidden_size, "state": "previous_input",
            "tensors": tuple(self.prefix + "mu." + name for name in self.BLENDS)}), compute_dtype)
        self.w = {}
        self.decay_bias = self.bonus = self.norm = None

    def cache_need(self):
        return (StateNeed((self.heads, self.dim, self.dim), torch.float32, "state"), self.blend.state_need())

    def tensors(self):
        p, h, n = self.prefix, self.hidden_size, self.inner
        out = {p + name: TensorSpec((n, h)) for name in ("r", "k", "v", "g")}
        out[p + "o"] = TensorSpec((h, n))
        out[p + "w0"] = TensorSpec((n,), init="bias")
        out[p + "u"] = TensorSpec((self.heads, self.dim), init="bias")
        out[p + "norm"] = TensorSpec((n,), init="norm")
        out[p + "w1"] = TensorSpec((self.default_rank, h), flexible=(0,))
        out[p + "w2"] = TensorSpec((n, self.default_rank), flexible=(1,))
        out.update(self.blend.tensors())
        return out

    def load(self, tensors, device):
        p = self.prefix
        if tensors[p + "w1"].shape[0] != tensors[p + "w2"].shape[1]:
            raise ValueError(f"{p}w1 and {p}w2 disagree on the decay's bottleneck width")
        for name in ("r", "k", "v", "g", "o", "w1", "w2"):
            self.w[name] = self._to_compute(tensors[p + name], device)
        self.decay_bias = _float(tensors[p + "w0"], device)
        self.bonus = _float(tensors[p + "u"], device).reshape(-1)
        self.norm = _float(tensors[p + "norm"], device)
        self.blend.load(tensors, device)

    def forward(self, x, ctx, view, writes_cache):
        k = ops.current()
        xr, xk, xv, xg, xw = self.blend.forward(x, ctx, view)
        f32 = torch.float32
        r = k.linear(xr, self.w["r"], out_dtype=f32)
        key = k.linear(xk, self.w["k"], out_dtype=f32)
        value = k.linear(xv, self.w["v"], out_dtype=f32)
        gate = k.linear(xg, self.w["g"], out_dtype=f32)
        decay = k.linear(k.tanh_(k.linear(xw, self.w["w1"])), self.w["w2"], out_dtype=f32)
        mixed = k.bonus_recurrence(r, key, value, decay, gate, self.decay_bias, self.bonus, self.norm, self.eps,
                                   view.states["state"], ctx, self.heads, self.dim, self.compute_dtype)
        return k.linear(mixed, self.w["o"], out_dtype=f32)


class HGRN2Mixer(Mixer):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.heads = int(a["heads"])
        self.dim = int(a["dim"])
        self.vdim = int(a["vdim"])
        self.eps = float(a["eps"])
        self.w_qfv = self.w_o = self.forget_bias = self.lower = self.norm = None

    def cache_need(self):
        return StateNeed((self.heads, self.dim, self.vdim), torch.float32, "state")

    def tensors(self):
        p, h, n = self.prefix, self.hidden_size, self.heads * self.dim
        return {p + "q": TensorSpec((n, h)), p + "f": TensorSpec((n, h)), p + "f.b": TensorSpec((n,), init="bias"),
                p + "lower": TensorSpec((n,), init="unit"), p + "v": TensorSpec((self.heads * self.vdim, h)),
                p + "norm": TensorSpec((self.vdim,), init="norm"), p + "o": TensorSpec((h, self.heads * self.vdim))}

    def load(self, tensors, device):
        p = self.prefix
        # one product yields [q | f | v]
        self.w_qfv = self._to_compute(torch.cat([tensors[p + "q"], tensors[p + "f"], tensors[p + "v"]], dim=0), device)
        self.w_o = self._to_compute(tensors[p + "o"], device)
        self.forget_bias = _float(tensors[p + "f.b"], device)
        self.lower = _float(tensors[p + "lower"], device)
        self.norm = _float(tensors[p + "norm"], device)

    def forward(self, x, ctx, view, writes_cache):
        k = ops.current()
        n = self.heads * self.dim
        qfv = k.linear(x, self.w_qfv, out_dtype=torch.float32)
        mixed = k.forget_gate_recurrence(qfv[:, :n], qfv[:, n:2 * n], qfv[:, 2 * n:], self.forget_bias, self.lower,
                                         self.norm, self.eps, view.states["state"], ctx, self.heads, self.dim,
                                         self.vdim, self.compute_dtype)
        return k.linear(mixed, self.w_o, out_dtype=torch.float32)


register_part("mixer", "wkv", WKVMixer)
register_part("mixer", "hgrn2", HGRN2Mixer)
