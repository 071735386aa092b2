"""A selective state-space layer with a scalar decay per head (the "state-space duality" form), as
a mixer.

One stacked projection of the input gives [z | x | B | C | dt]: inner = heads * vdim gate columns,
inner value columns, groups * state columns each for B and C, one step column per head. x, B and C
together pass a causal convolution per channel (taps and a bias per channel, the last tap the current
token's) and SiLU. dt <- softplus(dt + dt_bias). Per head h, which reads the B and C of group
h // (heads / groups):

    S_t = exp(-exp(A_h) dt_t) S_(t-1) + dt_t B_t x_t^T        S: [state, vdim], float32
    y_t = S_t^T C_t + D_h x_t

The heads side by side are multiplied by silu(z), RMS-normed in `norm_groups` equal parts (each by
its own root mean square), multiplied by a gain and projected back. A request keeps S and the last
taps - 1 inputs of the convolution in its state slot, zero at admission. Everything from dt on is
float32; the projection, the convolution and its activation are in the compute dtype.

The recurrence is the package's linear recurrence with k = B, q = C, v = x, a decay and an input
weight per token, and groups of heads sharing q and k (`ops.linear_recurrence(qk_share=)`).
"""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, Mixer, StateSpec, StepContext, register_part
from atomserve_b200.parts.spec import TensorSpec


class SelectiveStateSpace(Mixer):
    state_in_graphs = True  # the states are touched by this mixer's kernels alone, through ctx.state_slots

    def __init__(self, hidden_size: int, prefix: str, heads: int, vdim: int, state: int, groups: int, conv: int,
                 norm_groups: int, eps: float):  # fmt: skip
        if heads % groups or (heads * vdim) % norm_groups or conv < 1:
            raise ValueError(f"{heads} heads in {groups} groups, {heads * vdim} columns normed in {norm_groups} parts, {conv} taps")
        self.hidden_size, self.prefix = hidden_size, prefix
        self.heads, self.vdim, self.state, self.groups, self.taps = heads, vdim, state, groups, conv
        self.norm_groups, self.eps = norm_groups, float(eps)
        self.inner = heads * vdim
        self.channels = self.inner + 2 * groups * state  # what the convolution runs over: x, B, C
        self.in_proj = self.o_proj = None

    def state_specs(self) -> list[StateSpec]:
        return [StateSpec("s", (self.heads, self.state, self.vdim), torch.float32),
                StateSpec("conv", (self.taps - 1, self.channels), torch.float32)]  # fmt: skip

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, H = self.prefix, self.hidden_size, self.heads
        return [
            TensorSpec(p + "in", (2 * self.inner + 2 * self.groups * self.state + H, d)),
            TensorSpec(p + "conv", (self.channels, self.taps), kind="gain", init="normal"),
            TensorSpec(p + "conv.b", (self.channels,), kind="gain", init="normal"),
            TensorSpec(p + "dt_bias", (H,), kind="gain", init="normal"),
            TensorSpec(p + "A_log", (H,), kind="gain", init="normal"),
            TensorSpec(p + "D", (H,), kind="gain", init="gain"),
            TensorSpec(p + "norm", (self.inner,), kind="gain", init="gain"),
            TensorSpec(p + "o", (d, self.inner)),
        ]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p = self.prefix
        self.in_proj, self.o_proj = tensors[p + "in"], tensors[p + "o"]
        self.conv_taps, self.conv_bias = tensors[p + "conv"].contiguous(), tensors[p + "conv.b"]
        self.dt_bias, self.a_log, self.skip, self.gain = tensors[p + "dt_bias"], tensors[p + "A_log"], tensors[p + "D"], tensors[p + "norm"]

    def mixed(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None) -> torch.Tensor:
        """The gated, normed heads side by side, [T, inner], before the output projection."""
        inner, GN = self.inner, self.groups * self.state
        proj = ops.linear(h, self.in_proj)
        xbc, decay, weight = ops.conv_steps(proj, inner, 2 * inner + 2 * GN, self.conv_taps, self.conv_bias, cache.state["conv"],
                                            self.dt_bias, self.a_log, ctx.state_slots, ctx.req_q_start, ctx.num_requests)  # fmt: skip
        ops.conv_state_update(cache.state["conv"], proj, inner, ctx.state_slots, ctx.req_q_start, ctx.num_requests)
        # long portions are cut into segments that run side by side; the cut is made once per step
        # and shared by the step's recurrent layers
        if "lightning_segments" not in ctx.plans:
            ctx.plans["lightning_segments"] = ops.plan_segments(ctx.host_q_lens, proj.device) if ctx.host_q_lens else None
        y, _ = ops.linear_recurrence(xbc, inner + GN, inner, 0, cache.state["s"], ctx.state_slots, ctx.req_q_start,
                                     ctx.num_requests, token_decay=decay, token_gain=weight,
                                     qk_share=self.heads // self.groups, segments=ctx.plans["lightning_segments"])  # fmt: skip
        return ops.gate_group_norm(y, xbc[:, :inner], proj[:, :inner], self.skip, self.gain, self.norm_groups, self.vdim, self.eps)

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext,
                cache: CacheView | None, write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        # without a residual (a block that sums in float32 itself) the product stays float32
        return ops.linear(self.mixed(h, ctx, cache), self.o_proj, residual, out_dtype=torch.float32 if residual is None else None)

    def forward_for_stream(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool = True):
        """mix(h) for a block that adds it to a float32 stream itself: float32, or the output
        projection's partial sums for the norm that follows to add up (`ops.linear_for_stream`)."""
        return ops.linear_for_stream(self.mixed(h, ctx, cache), self.o_proj)


register_part("mixer", "selective_state_space", SelectiveStateSpace)
