"""Token shift: y_t = a_t + (a_{t-1} - a_t) * c, channel by channel, with a_{-1} = 0.

The previous token's row belongs to the request: the last row of every step is kept in a 32-bit
state of the request's slot and is the "previous row" of the next step's first token, so that the
result does not depend on how a prompt is cut.  Several coefficient vectors may be applied to the
same rows at once (``extra``): a mixer that blends its input differently for each of its
projections asks for all blends in one pass.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Shift, StateNeed, TensorSpec, register_part


class TokenShift(Shift):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.size = int(self.args["hidden_size"])
        self.state_name = str(self.args.get("state", "shift"))
        # checkpoint names of the coefficient vectors, in the order of the returned blends
        names = self.args.get("tensors") or (self.args.get("tensor") or self.prefix + "shift",)
        self.names = tuple(names)
        self.coefficients: torch.Tensor | None = None     # float32 [n, size]

    def state_need(self):
        return StateNeed((self.size,), torch.float32, self.state_name)

    def tensors(self):
        return {name: TensorSpec((self.size,), init="unit") for name in self.names}

    def load(self, tensors, device):
        self.coefficients = torch.stack([tensors[name].float() for name in self.names]).to(device).contiguous()

    def forward(self, x, ctx, view, out_dtype=None):
        """x: float32 [rows, size] -> [n, rows, size] in ``out_dtype`` (default: the compute dtype)."""
        return ops.current().token_shift(x, self.coefficients, view.states[self.state_name], ctx,
                                         out_dtype or self.compute_dtype)


register_part("shift", "token_shift", TokenShift)
