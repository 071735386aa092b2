"""Linear attention with a fixed decay per head ("lightning attention") as a mixer.

Per head, S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, with q, k and v the activated
projections of the input; the heads' outputs side by side are RMS-normed together, multiplied by
a sigmoid gate projected from the same input, and projected back. The state S ([dim, vdim] per
head, float32) is all the mixer keeps of a request: it lives in the request's state slot, zero
at admission, and is carried from step to step. Heads, sizes, decays, eps and the activation
are parameters. So are, for the form known as retention: a position encoding that rotates q and k
(`position`), a scale on k after the rotation (`k_scale`), a norm of each head by itself instead
of all together (`head_norm="each"`), no gain on that norm (`norm_gain=False`) and a SiLU gate
instead of a sigmoid (`gate="silu"`).
"""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, Mixer, StateSpec, StepContext, build_part, register_part
from atomserve_b200.parts.spec import PartSpec, TensorSpec


class LightningAttention(Mixer):
    state_in_graphs = True  # the state is touched by this mixer's kernel alone, through ctx.state_slots

    def __init__(self, hidden_size: int, prefix: str, heads: int, dim: int, vdim: int, decay: list[float], eps: float,
                 activation: str = "silu", position: PartSpec | None = None, k_scale: float = 1.0,
                 head_norm: str = "all", norm_gain: bool = True, gate: str = "sigmoid"):  # fmt: skip
        if head_norm not in ("all", "each") or gate not in ("sigmoid", "silu"):
            raise ValueError(f"head_norm {head_norm!r} is 'all' or 'each', gate {gate!r} 'sigmoid' or 'silu'")
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        if activation not in ("silu", "none"):
            raise ValueError(f"activation {activation!r} is neither 'silu' nor 'none'")
        self.hidden_size, self.prefix = hidden_size, prefix
        self.heads, self.dim, self.vdim, self.eps = heads, dim, vdim, float(eps)
        self.decay_values, self.activation = [float(d) for d in decay], activation
        self.position = build_part("position", position, hidden_size) if position else None
        self.k_scale, self.head_norm, self.norm_gain, self.gate = float(k_scale), head_norm, norm_gain, gate
        self.plain = position is None and k_scale == 1.0 and head_norm == "all" and norm_gain and gate == "sigmoid"
        self.in_proj = self.o_proj = self.gain = self.decay = None

    def state_specs(self) -> list[StateSpec]:
        return [StateSpec("s", (self.heads, self.dim, self.vdim), torch.float32)]

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, qk, vg = self.prefix, self.hidden_size, self.heads * self.dim, self.heads * self.vdim
        return [
            TensorSpec(p + "q", (qk, d)), TensorSpec(p + "k", (qk, d)), TensorSpec(p + "v", (vg, d)),
            TensorSpec(p + "g", (vg, d)), TensorSpec(p + "o", (d, vg)),
        ] + ([TensorSpec(p + "norm", (vg,), kind="gain", init="gain")] if self.norm_gain else [])  # fmt: skip

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p = self.prefix
        # q, k, v and the gate stacked along the output rows: one product instead of four
        self.in_proj = torch.cat([tensors[p + n] for n in "qkvg"]).contiguous()
        self.o_proj, self.gain = tensors[p + "o"], (tensors[p + "norm"] if self.norm_gain else None)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.o_proj.device)
        if self.position is not None:
            self.position.prepare(self.o_proj.device)
            rotary = self.position.fused_rotary()
            if rotary is None or rotary.pairing != "half" or rotary.magnitude != 1.0:
                raise NotImplementedError("the recurrence's kernel turns pairs (i, i + rotary_dim / 2) by position x frequency only")

    def input_weights(self) -> torch.Tensor:
        """The stacked input projection, for a mixer that runs this one beside another and
        multiplies once for both (`mixed_from` then reads this one's columns of the product)."""
        return self.in_proj

    def mixed(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None) -> torch.Tensor:
        """The gated, normed heads side by side, [T, heads * vdim], before the output projection."""
        return self.mixed_from(ops.linear(h, self.in_proj), 0, ctx, cache)

    def mixed_from(self, proj: torch.Tensor, col: int, ctx: StepContext, cache: CacheView | None) -> torch.Tensor:
        """The same from a product that holds this mixer's projection in the columns from `col`."""
        qk, vg = self.heads * self.dim, self.heads * self.vdim
        # long portions are cut into segments that run side by side; the cut is made once per step
        # and shared by the step's layers
        if "lightning_segments" not in ctx.plans:
            ctx.plans["lightning_segments"] = ops.plan_segments(ctx.host_q_lens, proj.device) if ctx.host_q_lens else None
        gate = proj[:, col + 2 * qk + vg : col + 2 * qk + 2 * vg]
        if self.plain:
            o = ops.lightning_attention(proj, col, col + qk, col + 2 * qk, cache.state["s"], ctx.state_slots, ctx.req_q_start,
                                        self.decay, ctx.num_requests, activation=self.activation == "silu",
                                        segments=ctx.plans["lightning_segments"])  # fmt: skip
            return ops.gated_rms_norm(o, gate, self.gain, self.eps)
        rotary = self.position.fused_rotary() if self.position is not None else None
        table = None
        if rotary:  # the step's cosines and sines, made once for all layers that turn by these frequencies
            key = f"rotary_table:{getattr(self.position, 'theta', id(self.position))}:{rotary.rotary_dim}"
            if key not in ctx.plans:
                ctx.plans[key] = ops.rotary_table(ctx.positions[: proj.shape[0]], rotary.inv_freq)
            table = ctx.plans[key]
        o, _ = ops.linear_recurrence(proj, col, col + qk, col + 2 * qk, cache.state["s"], ctx.state_slots, ctx.req_q_start,
                                     ctx.num_requests, decay=self.decay, k_scale=self.k_scale,
                                     positions=ctx.positions if rotary else None, inv_freq=rotary.inv_freq if rotary else None,
                                     rotary_dim=rotary.rotary_dim if rotary else 0, table=table, activation=self.activation == "silu",
                                     segments=ctx.plans["lightning_segments"])  # fmt: skip
        return ops.head_norm_gate(o, gate, self.heads if self.head_norm == "each" else 1, gain=self.gain, eps=self.eps,
                                  gate_activation=self.gate)  # fmt: skip

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext,
                cache: CacheView | None, write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        # without a residual (a block that sums in float32 itself) the product stays float32
        return ops.linear(self.mixed(h, ctx, cache), self.o_proj, residual, out_dtype=torch.float32 if residual is None else None)

    def forward_for_stream(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool = True):
        """mix(h) for a block that adds it to a float32 stream and norms the sum at once: float32, or
        the output projection's partial sums for that norm to add up (`ops.linear_for_stream`)."""
        return ops.linear_for_stream(self.mixed(h, ctx, cache), self.o_proj)

    def forward_from(self, proj: torch.Tensor, col: int, ctx: StepContext, cache: CacheView | None) -> torch.Tensor:
        """mix(h) as float32, from a product that holds this mixer's projection from column `col`."""
        return ops.linear(self.mixed_from(proj, col, ctx, cache), self.o_proj, out_dtype=torch.float32)


register_part("mixer", "lightning_attention", LightningAttention)
