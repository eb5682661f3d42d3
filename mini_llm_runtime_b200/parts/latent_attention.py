"""Attention whose queries, keys and values are made from low-rank latents.

With h the mixer's input, per token:

    cq = rms_norm(Wdq h) * nq                      query latent [q_rank]
    q  = Wuq cq                                    per head [dim plain | rot_dim to be turned]
    [c_raw | r_raw] = Wdkv h                       kv_rank + rot_dim numbers
    c  = rms_norm(c_raw) * nc                      key/value latent [kv_rank]
    r  = turn(r_raw, position)                     one turned key part for all heads

    score(i, j, head) = (q_plain . (Wuk[head] c_j) + turn(q_rot, i) . r_j) * scale
    out(i, head)      = sum_j softmax_j(score) * (Wuv[head] c_j)

followed by a sigmoid gate computed from h (one number per output channel, or one per head) and
the output projection.  Only [c | r] is cached, one row per token shared by all heads: the
queries are carried into the latent space (Wuk[head]^T q_plain), the attention sums latents, and
Wuv[head] is applied to the sum.  Variants, all parameters of the spec: the pair layout of the
rotation (``rope_layout``: ``half`` or ``interleaved``), a sliding window (``window`` keys
including the token itself; 0: all earlier keys), a learned per-head sink in the softmax
denominator (``sink``), and the gate's granularity (``gate``: ``channel`` or ``head``).

32-bit: both RMS norms, angles and rotation, scores and softmax, the latent sums, the gate.  In
bfloat16 the products' operands and the cached rows are bfloat16.
"""

from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from ..ops import AttentionBatch
from .base import KVCacheNeed, Mixer, TensorSpec, build_part, register_part


class LatentAttention(Mixer):
    graph_safe = True
    plan_key = "paged_attention"

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.heads = int(a["heads"])
        self.dim = int(a["dim"])
        self.rot_dim = int(a["rot_dim"])
        self.vdim = int(a["vdim"])
        self.kv_rank = int(a["kv_rank"])
        self.q_rank = int(a["q_rank"])
        self.scale = float(a["scale"])
        self.eps = float(a["eps"])
        self.window = int(a.get("window") or 0)
        self.has_sink = bool(a.get("sink", False))
        self.gate_kind = str(a.get("gate", "channel"))
        if self.gate_kind not in ("channel", "head"):
            raise ValueError(f"unknown gate granularity {self.gate_kind!r}; known: channel, head")
        rope_dims = int(a.get("rope_dims", self.rot_dim))
        if rope_dims % 2 or not 0 < rope_dims <= self.rot_dim:
            raise ValueError("the rotation covers an even number of entries, at most rot_dim")
        self.position = build_part("position", PartSpec("rope_pairs", {
            "head_dim": rope_dims, "theta": float(a["rope_base"]), "layout": a.get("rope_layout", "half")}), compute_dtype)
        self.gate_width = self.heads if self.gate_kind == "head" else self.heads * self.vdim
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = None
        self.q_norm = self.c_norm = self.sink = None

    def cache_need(self):
        return KVCacheNeed(1, self.kv_rank + self.rot_dim, self.window or None, value_dim=0)

    def tensors(self):
        p, h = self.prefix, self.hidden_size
        out = {p + "dq": TensorSpec((self.q_rank, h)), p + "dq.norm": TensorSpec((self.q_rank,), init="norm"),
               p + "uq": TensorSpec((self.heads * (self.dim + self.rot_dim), self.q_rank)),
               p + "dkv": TensorSpec((self.kv_rank + self.rot_dim, h)),
               p + "dkv.norm": TensorSpec((self.kv_rank,), init="norm"),
               p + "uk": TensorSpec((self.heads * self.dim, self.kv_rank)),
               p + "uv": TensorSpec((self.heads * self.vdim, self.kv_rank)),
               p + "g": TensorSpec((self.gate_width, h)), p + "o": TensorSpec((h, self.heads * self.vdim))}
        if self.has_sink:
            out[p + "sink"] = TensorSpec((self.heads,), init="bias")
        return out

    def load(self, tensors, device):
        p = self.prefix
        # one product yields [query latent | key/value latent | key part to be turned | gate]
        self.w_down = self._to_compute(torch.cat([tensors[p + "dq"], tensors[p + "dkv"], tensors[p + "g"]], dim=0), device)
        for name in ("uq", "uk", "uv", "o"):
            setattr(self, "w_" + name, self._to_compute(tensors[p + name], device))
        self.q_norm = tensors[p + "dq.norm"].to(device=device, dtype=torch.float32).contiguous()
        self.c_norm = tensors[p + "dkv.norm"].to(device=device, dtype=torch.float32).contiguous()
        if self.has_sink:
            self.sink = tensors[p + "sink"].to(device=device, dtype=torch.float32).contiguous()
        self.position.load({}, device)

    def step_plan(self, host):
        return ops.current().plan_attention(host.lengths, host.position_start)

    def _batch(self, ctx, view) -> AttentionBatch:
        batch = view.shared.get("attention_batch")
        if batch is None:
            arrays, counts = ctx.plans.get(self.plan_key, ({}, {}))
            batch = AttentionBatch(
                seg_q_start=ctx.seg_q_start, seg_q_len=ctx.seg_q_len, seg_pos0=ctx.seg_pos0, seg_slot=ctx.seg_slot,
                block_table=view.block_table, num_segments=ctx.num_segments, max_q_len=ctx.max_q_len,
                max_kv_len=ctx.max_kv_len, plan=arrays, counts=counts)
            view.shared["attention_batch"] = batch
        return batch

    def forward(self, x, ctx, view, writes_cache):
        k = ops.current()
        frequencies, interleaved = self.position.rotary_frequencies(), self.position.interleaved
        down = k.linear(x, self.w_down, out_dtype=torch.float32)
        gate_at = self.q_rank + self.kv_rank + self.rot_dim
        q_latent = k.latent_prepare(down, 0, self.q_rank, self.q_rank, self.kv_rank, self.rot_dim, self.q_norm,
                                    self.c_norm, self.eps, ctx.positions, frequencies, interleaved, view.slots,
                                    view.k_pool, writes_cache)
        q = k.linear(q_latent, self.w_uq, out_dtype=torch.float32)
        absorbed = k.absorb_queries(q, self.w_uk, self.heads, self.dim, self.rot_dim, self.kv_rank, ctx.positions,
                                    frequencies, interleaved)
        mixed = k.latent_attention(absorbed, view.k_pool, self._batch(ctx, view), self.heads, self.kv_rank,
                                   self.rot_dim, self.scale, self.window, self.sink)
        gated = k.latent_values(mixed, self.w_uv, self.heads, self.vdim, self.kv_rank,
                                down[:, gate_at:gate_at + self.gate_width], self.gate_kind == "head")
        return k.linear(gated, self.w_o, out_dtype=torch.float32)


register_part("mixer", "latent_attention", LatentAttention)
