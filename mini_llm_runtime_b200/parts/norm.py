"""RMSNorm: y = w * x * rsqrt(mean(x^2) + eps), all in float32, eps inside the root, no centering
and no bias (reference: src/mini_llm_runtime/qwen_model_runner.py:22-26).  The reference casts the
normalised row back to the model dtype before multiplying by w; here the product is taken in
float32 and rounded once."""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, TensorSpec, register_part


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.size = int(self.args["size"])
        self.eps = float(self.args["eps"])
        self.weight: torch.Tensor | None = None
        self.folded = False       # True once the weight lives in the matrix that follows

    def tensors(self):
        return {self.prefix + "weight": TensorSpec((self.size,), init="norm")}

    def load(self, tensors, device):
        self.weight = self._keep_precision(tensors[self.prefix + "weight"], device)

    def fold(self):
        self.folded = True
        return self.weight, self.eps

    def forward(self, x):
        return ops.current().rms_norm(x, None if self.folded else self.weight, self.eps)

    def add_forward(self, residual, delta):
        return ops.current().add_rms_norm(residual, delta, None if self.folded else self.weight, self.eps)


class ScalarRMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * g with a single learned number g for the whole row.  It reads
    a 32-bit residual stream and hands out rows in the compute dtype (``forward``), or both those and
    the 32-bit rows (``forward_both``) for what continues in 32-bit.  The checkpoint tensor (a scalar)
    is named by the spec (``tensor``)."""

    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.eps = float(self.args["eps"])
        self.tensor = self.args.get("tensor") or self.prefix + "weight"
        self.gain: torch.Tensor | None = None

    def tensors(self):
        return {self.tensor: TensorSpec((), init="norm")}

    def load(self, tensors, device):
        self.gain = tensors[self.tensor].to(device=device, dtype=torch.float32).reshape(1).contiguous()

    def forward(self, x):
        return ops.current().scalar_rms_norm(x, self.gain, self.eps, self.compute_dtype)

    def forward_both(self, x):
        return ops.current().scalar_rms_norm(x, self.gain, self.eps, self.compute_dtype, want_float=True)


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "scalar_rms_norm", ScalarRMSNorm)
