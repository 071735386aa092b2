"""Dense SwiGLU feed-forward: residual + down( silu(gate(h)) * up(h) ), no biases
(atomserve/model.py:339-360)."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import FeedForward, Norm, StepContext, register_part
from atomserve_b200.parts.spec import TensorSpec


class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, prefix: str, intermediate_size: int):
        self.hidden_size, self.prefix, self.intermediate_size = hidden_size, prefix, intermediate_size
        self.gate_up_proj = self.down_proj = None
        self.fused = False

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, i = self.prefix, self.hidden_size, self.intermediate_size
        return [
            TensorSpec(p + "gate_proj.weight", (i, d)),
            TensorSpec(p + "up_proj.weight", (i, d)),
            TensorSpec(p + "down_proj.weight", (d, i)),
        ]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p = self.prefix
        gate, up = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        self.fused = gate.is_cuda and ops.swiglu_fusable(gate)
        if self.fused:
            # rows alternate gate_i, up_i: the tensor-core GEMM applies SiLU * up in its epilogue
            self.gate_up_proj = ops.interleave_gate_up(gate, up)
        else:
            # gate rows first, then up rows (atomserve/loader.py:121)
            self.gate_up_proj = torch.cat([gate, up]).contiguous()
        self.down_proj = tensors[p + "down_proj.weight"]

    def hidden(self, h: torch.Tensor) -> torch.Tensor:
        if self.fused:
            return ops.linear_swiglu(h, self.gate_up_proj)
        return ops.silu_mul(ops.linear(h, self.gate_up_proj))

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ops.linear(self.hidden(h), self.down_proj, residual)

    def forward_then(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext,
                     then: Norm) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
        after_linear = getattr(then, "after_linear", None)
        if after_linear is None:
            return super().forward_then(h, residual, ctx, then)
        return after_linear(self.hidden(h), self.down_proj, residual)


class GatedMLP(FeedForward):
    """down(act(gate h + b_gate) * (up h + b_up)) + b_down with act "silu", "gelu_tanh" or "gelu" and
    optional biases; tensors `gate`, `up`, `down` and their `.b`. The down projection's bias is
    `output_bias`: a block that norms the sublayer's output adds it in that norm's kernel."""

    def __init__(self, hidden_size: int, prefix: str, intermediate_size: int, activation: str = "gelu_tanh", biases: bool = True):
        if activation not in ops.sandwich.GLU_ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {sorted(ops.sandwich.GLU_ACTIVATIONS)}")
        self.hidden_size, self.prefix, self.intermediate_size = hidden_size, prefix, intermediate_size
        self.activation, self.biases = activation, biases
        self.gate_up = self.down = self.gate_up_bias = self.output_bias = None
        self.fused = False

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, i = self.prefix, self.hidden_size, self.intermediate_size
        specs = [TensorSpec(p + "gate", (i, d)), TensorSpec(p + "up", (i, d)), TensorSpec(p + "down", (d, i))]
        if self.biases:
            specs += [TensorSpec(p + "gate.b", (i,), kind="gain", init="normal"), TensorSpec(p + "up.b", (i,), kind="gain", init="normal"),
                      TensorSpec(p + "down.b", (d,), kind="gain", init="normal")]  # fmt: skip
        return specs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p = self.prefix
        gate, up = tensors[p + "gate"], tensors[p + "up"]
        self.fused = gate.is_cuda and ops.swiglu_fusable(gate)
        if self.fused:
            # rows alternate gate_i, up_i (the biases too): the tensor-core GEMM adds the biases and
            # applies act(gate) * up in its epilogue
            self.gate_up = ops.interleave_gate_up(gate, up)
        else:
            self.gate_up = torch.cat([gate, up]).contiguous()  # one product for both, gate rows first
        self.down = tensors[p + "down"]
        if self.biases:
            b_gate, b_up = tensors[p + "gate.b"], tensors[p + "up.b"]
            self.gate_up_bias = (torch.stack([b_gate, b_up], dim=1).reshape(-1) if self.fused else torch.cat([b_gate, b_up])).contiguous()
            self.output_bias = tensors[p + "down.b"]

    def inner(self, h: torch.Tensor) -> torch.Tensor:
        if self.fused:
            return ops.linear_glu(h, self.gate_up, self.gate_up_bias, self.activation)
        return ops.bias_glu(ops.linear(h, self.gate_up), self.gate_up_bias, self.activation)

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext) -> torch.Tensor:
        out = ops.linear(self.inner(h), self.down, None, out_dtype=torch.float32)
        if self.output_bias is not None:
            out += self.output_bias
        return out if residual is None else residual + out.to(residual.dtype)

    def forward_for_stream(self, h: torch.Tensor, ctx: StepContext):
        """ff(h) without the output bias, for a block that adds it to a float32 stream itself:
        float32, or the down projection's partial sums (`ops.linear_for_stream`)."""
        return ops.linear_for_stream(self.inner(h), self.down)


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "gated_mlp", GatedMLP)
