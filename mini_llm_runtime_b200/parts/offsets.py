"""Learned vectors added to the residual stream at places the run order names.

A model that passes a run of its layers several times with the same weights tells the passes apart
by a vector added to every row before each pass: row t of one table [passes, width] before pass t.
The table is 32-bit on the device (it joins a 32-bit stream); the run step names the row.
"""

from __future__ import annotations

import torch

from .base import StreamOffsets, TensorSpec, register_part


class LearnedOffsets(StreamOffsets):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.rows = int(self.args["rows"])
        self.size = int(self.args["size"])
        self.tensor = self.args.get("tensor") or self.prefix + "weight"
        self.table: torch.Tensor | None = None

    def tensors(self):
        return {self.tensor: TensorSpec((self.rows, self.size), init="bias")}

    def load(self, tensors, device):
        self.table = tensors[self.tensor].to(device=device, dtype=torch.float32).contiguous()

    def vector(self, row):
        if not 0 <= row < self.rows:
            raise IndexError(f"offset row {row} is outside the table's {self.rows} rows")
        return self.table[row]


register_part("offset", "learned_offsets", LearnedOffsets)
