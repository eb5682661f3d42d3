"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(reference: src/mini_llm_runtime/qwen_model_runner.py:215-217).  gate and up are stacked into one
[2*intermediate, hidden] matrix at load time so that one product feeds the activation.  When the
intermediate width is a multiple of 64 the rows are interleaved in blocks (64 gate rows, then the
64 up rows of the same outputs), which lets the tensor-core kernel apply the activation in its
epilogue; otherwise all gate rows come first."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_part


class SwiGLU(FeedForward):
    graph_safe = True
    supports_norm_fusion = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.hidden_size = int(self.args["hidden_size"])
        self.intermediate_size = int(self.args["intermediate_size"])
        self.w_gate_up = self.w_down = None
        self.block = self.intermediate_size   # gate/up interleaving of w_gate_up
        self.input_norm_eps: float | None = None

    def tensors(self):
        p = self.prefix
        return {
            p + "gate_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            p + "up_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            p + "down_proj.weight": TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def load(self, tensors, device):
        p = self.prefix
        gate, up = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        if self.intermediate_size % 64 == 0:
            self.block = 64
            stacked = torch.cat([gate.view(-1, 64, self.hidden_size), up.view(-1, 64, self.hidden_size)], dim=1)
            stacked = stacked.reshape(2 * self.intermediate_size, self.hidden_size)
        else:
            stacked = torch.cat([gate, up], dim=0)
        self.w_gate_up = self._to_compute(stacked, device)
        self.w_down = self._to_compute(tensors[p + "down_proj.weight"], device)

    def absorb_input_norm(self, weight, eps):
        folded = self.w_gate_up.float() * weight.to(self.w_gate_up.device).float()[None, :]
        self.w_gate_up = folded.to(self.compute_dtype).contiguous()
        self.input_norm_eps = float(eps)

    def forward(self, x, ctx, raw_input=False, residual=None):
        k = ops.current()
        hidden = k.linear_swiglu(x, self.w_gate_up, self.block,
                                 rms_eps=self.input_norm_eps if raw_input else None)
        return k.linear(hidden, self.w_down, residual=residual)


class GatedMLP(FeedForward):
    """down(act(gate(x)) * up(x)) without biases, ``activation`` being ``silu`` or ``gelu_tanh``
    (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))); or, with ``activation="clamped_swish"``,
    down(g * sigmoid(slope * g) * (u + 1)) where g = min(gate(x), limit) and u = clamp(up(x), -limit,
    limit) (``limit`` from the spec, ``slope`` 1.702 unless given).  The result leaves in 32-bit floats, for
    arrangements that sum into a 32-bit stream.  ``names`` gives the three checkpoint names after
    the prefix.  gate and up are stacked like SwiGLU's."""

    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.hidden_size = int(self.args["hidden_size"])
        self.intermediate_size = int(self.args["intermediate_size"])
        self.activation = str(self.args.get("activation", "silu"))
        if self.activation not in ("silu", "gelu_tanh", "clamped_swish"):
            raise ValueError(f"unknown gate activation {self.activation!r}")
        self.limit = float(self.args.get("limit", 0.0))
        self.slope = float(self.args.get("slope", 1.702))
        if self.activation == "clamped_swish" and not self.limit > 0:
            raise ValueError("the clamped gate needs a positive limit")
        self.names = tuple(self.args.get("names") or ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))
        self.w_gate_up = self.w_down = None
        self.block = self.intermediate_size

    def tensors(self):
        gate, up, down = (self.prefix + name for name in self.names)
        return {gate: TensorSpec((self.intermediate_size, self.hidden_size)),
                up: TensorSpec((self.intermediate_size, self.hidden_size)),
                down: TensorSpec((self.hidden_size, self.intermediate_size))}

    def load(self, tensors, device):
        gate, up, down = (tensors[self.prefix + name] for name in self.names)
        if self.intermediate_size % 64 == 0:
            self.block = 64
            stacked = torch.cat([gate.view(-1, 64, self.hidden_size), up.view(-1, 64, self.hidden_size)], dim=1)
            stacked = stacked.reshape(2 * self.intermediate_size, self.hidden_size)
        else:
            stacked = torch.cat([gate, up], dim=0)
        self.w_gate_up = self._to_compute(stacked, device)
        self.w_down = self._to_compute(down, device)

    def forward(self, x, ctx):
        k = ops.current()
        if self.activation == "clamped_swish":
            hidden = k.linear_clamped_gate(x, self.w_gate_up, self.block, self.limit, self.slope)
        else:
            hidden = k.linear_gated(x, self.w_gate_up, self.block, self.activation)
        return k.linear(hidden, self.w_down, out_dtype=torch.float32)


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "gated_mlp", GatedMLP)
