"""A decoder put together from a ``ModelSpec``: embedding, blocks in their run order, final norm,
head.  This class is the same for every architecture; what differs is the spec.

It corresponds to the reference's ``QwenPrefillRunner`` (src/mini_llm_runtime/qwen_model_runner.py:
227-508) with its four entry points (prefill, prefill_batch, decode_one, decode_batch) replaced by
one ``forward`` over a ragged step batch.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.spec import ModelSpec
from ..parts.base import Block, KVCacheNeed, PendingDelta, StateNeed, TensorSpec, build_part, part_factory
from ..weights.loader import check_tensors


class DecoderModel:
    def __init__(self, spec: ModelSpec, compute_dtype: torch.dtype) -> None:
        if compute_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("the model computes in float32 or bfloat16")
        self.spec = spec
        self.compute_dtype = compute_dtype
        self.embedding = build_part("embedding", spec.embedding, compute_dtype)
        self.blocks: list[Block] = []
        for layer in spec.layers:
            block_cls = part_factory("block", layer.block)
            extras = {name: build_part(category, part_spec, compute_dtype)
                      for name, category, part_spec in layer.extra_parts}
            self.blocks.append(block_cls(
                build_part("mixer", layer.mixer, compute_dtype),
                None if layer.feed_forward is None else build_part("feed_forward", layer.feed_forward, compute_dtype),
                build_part("norm", layer.mixer_norm, compute_dtype),
                None if layer.feed_forward_norm is None else build_part("norm", layer.feed_forward_norm, compute_dtype),
                **({"extras": extras} if extras else {}),
            ))
        self.offsets = None if spec.offsets is None else build_part("offset", spec.offsets, compute_dtype)
        self.final_norm = build_part("norm", spec.final_norm, compute_dtype)
        self.head = build_part("head", spec.head, compute_dtype)
        self.device: torch.device | None = None

    # ------------------------------------------------------------------ weights
    def parts(self):
        yield self.embedding
        for block in self.blocks:
            yield from block.parts()
        if self.offsets is not None:
            yield self.offsets
        yield self.final_norm
        yield self.head

    def expected_tensors(self) -> dict[str, TensorSpec]:
        expected: dict[str, TensorSpec] = {}
        for part in self.parts():
            for name, tensor_spec in part.tensors().items():
                if name in expected and expected[name] != tensor_spec:
                    raise ValueError(f"two parts claim tensor {name!r} with different expectations")
                expected[name] = tensor_spec
        return expected

    def load(self, tensors: Mapping[str, torch.Tensor], device: torch.device | str) -> "DecoderModel":
        """Check ``tensors`` (as stored, on the CPU) against the parts and hand them over."""
        expected = self.expected_tensors()
        check_tensors(expected, tensors)
        self.device = torch.device(device)
        for part in self.parts():
            part.load(tensors, self.device)
        for block in self.blocks:
            block.finish_load(self.compute_dtype)
        return self

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> list:
        """What each cache entry must hold, taken from the layer of the run step that writes it: a
        ``KVCacheNeed``, a ``StateNeed``, a tuple of them, or None."""
        needs: list = [None] * self.spec.cache_entries
        for step in self.spec.run_order:
            need = self.blocks[step.layer].cache_need()
            if step.writes_cache:
                needs[step.cache] = need
            elif needs[step.cache] != need:
                raise ValueError(f"layer {step.layer} reads cache entry {step.cache}, whose layout "
                                 f"{needs[step.cache]} differs from what it needs ({need})")
        return needs

    # ------------------------------------------------------------------ forward
    def forward(self, ctx) -> torch.Tensor:
        """Run the step's rows through the model; float32 logits [wanted rows, vocab]."""
        if self.embedding.needs_positions:
            residual = self.embedding.forward(ctx.token_ids, ctx.positions)
        else:
            residual = self.embedding.forward(ctx.token_ids)
        pending = None
        for step in self.spec.run_order:
            view = ctx.cache_view(step.cache)
            block = self.blocks[step.layer]
            if step.offset_row is None:
                residual, pending = block.forward(residual, pending, ctx, view, step.writes_cache)
            elif block.takes_offset:
                residual, pending = block.forward(residual, pending, ctx, view, step.writes_cache,
                                                  offset=self.offsets.vector(step.offset_row))
            else:
                residual = self._settle(residual, pending)
                residual = ctx.ops.add_rows(residual, self.offsets.vector(step.offset_row))
                residual, pending = block.forward(residual, None, ctx, view, step.writes_cache)
        if ctx.num_wanted == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=residual.device)
        k = ctx.ops
        everything = getattr(ctx, "wanted_all_rows", False)      # every row in order (a decode step)
        rows = residual if everything else k.gather_rows(residual, ctx.wanted_rows)
        if pending is None:
            normed = self.final_norm.forward(rows)
        else:
            post = pending.norm if isinstance(pending, PendingDelta) else None
            delta = pending.tensor if isinstance(pending, PendingDelta) else pending
            delta = delta if everything else k.gather_rows(delta, ctx.wanted_rows)
            # the stream itself must stay as it is only if it is read again; it is not after the last layer
            normed = (self.final_norm.add_forward(rows, delta) if post is None
                      else self.final_norm.add_forward(rows, delta, post=post))
        return self.head.forward(normed, self.embedding)

    @staticmethod
    def _settle(residual, pending):
        """Add what is still pending into the stream."""
        if pending is None:
            return residual
        if isinstance(pending, PendingDelta):
            if pending.norm is not None:
                return pending.norm.add_into(residual, pending.tensor)
            pending = pending.tensor
        from .. import ops
        return ops.current().add_inplace(residual, pending)
