"""Transformations of the residual stream that a run order places between layers.

`MixWithInput`: x <- W [x ; x0] + step[number], with x0 what the embedding gave and `step` a table
of one vector per use: how a model that runs a stretch of its layers several times with the same
weights opens each pass. The product reads both streams in the compute dtype and leaves float32."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import StepContext, StreamStep, register_part
from atomserve_b200.parts.spec import TensorSpec


class MixWithInput(StreamStep):
    def __init__(self, hidden_size: int, prefix: str, uses: int, tensor: str | None = None, step_tensor: str | None = None):
        self.width, self.uses = hidden_size, int(uses)
        self.name, self.step_name = tensor or prefix + "in", step_tensor or prefix + "step"
        self.weight = self.steps = None
        self.dtype = torch.float32

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.width, 2 * self.width)),
                TensorSpec(self.step_name, (self.uses, self.width), kind="gain", init="normal")]  # fmt: skip

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight, self.steps = tensors[self.name], tensors[self.step_name].contiguous()

    def bind_dtype(self, dtype: torch.dtype) -> None:
        self.dtype = dtype

    def product(self, x: torch.Tensor, x0: torch.Tensor) -> torch.Tensor:
        """W [x ; x0] as float32 (the vector of the use is added by whoever norms the result)."""
        return ops.linear(ops.concat_cast(x, x0, self.dtype), self.weight, out_dtype=torch.float32)

    def forward(self, x: torch.Tensor, x0: torch.Tensor, number: int, ctx: StepContext) -> torch.Tensor:
        return self.forward_then(x, x0, number, ctx, None)[0]

    def forward_then(self, x: torch.Tensor, x0: torch.Tensor, number: int, ctx: StepContext, then):
        """(the new stream, what the block that follows reads first or None): where that block's
        first norm says how the block norms its input twice (`block_norms`), the kernel that adds
        the use's vector gives both norms as well."""
        if not 0 <= number < self.uses:
            raise ValueError(f"use {number} of a step table of {self.uses}")
        owner = getattr(then, "block_norms", None) if then is not None else None
        if owner is None:
            return ops.residual_dual_norm(None, self.product(x, x0), None, 1.0, None, None, 0.0, self.dtype, bias=self.steps[number])[0], None
        g1, g2, eps = owner()
        x, h1, h2 = ops.residual_dual_norm(None, self.product(x, x0), None, 1.0, g1, g2, eps, self.dtype, bias=self.steps[number])
        return x, (h1, h2)


register_part("stream_step", "mix_with_input", MixWithInput)
