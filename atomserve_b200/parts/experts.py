"""Feed-forwards beyond SwiGLU: a dense two-matrix GELU layer, routed experts with grouped
selection and an optional gated shared expert, and the feed-forward a layer does not have.

Routed experts: router logits z = Wr h in float32; scores sigmoid(z) (or a softmax); with
`groups` > 1 the experts form that many equal groups of neighbours, a group scores the sum of
its `group_top` largest scores and only the `keep` best groups' experts can be chosen; each
token takes the `top` largest allowed scores, weighted s / (sum s + 1e-20) * scale. An expert is
down(g sigmoid(slope g) (u + shift)) with g = min(gate h, limit), u = clamp(up h, -limit, limit).
A shared expert of the same form (own size and limit) runs for every token and is added, times
sigmoid(Wsg h) when it is gated. All of these are parameters.
"""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import FeedForward, StepContext, register_part
from atomserve_b200.parts.spec import TensorSpec


class GeluMLP(FeedForward):
    """down(act(up h)) with act the exact (erf) GELU, its tanh form, or (`activation="relu2"`) the
    squared ReLU; no biases."""

    def __init__(self, hidden_size: int, prefix: str, intermediate_size: int, tanh_form: bool = False,
                 activation: str | None = None):  # fmt: skip
        self.hidden_size, self.prefix, self.intermediate_size, self.tanh_form = hidden_size, prefix, intermediate_size, tanh_form
        self.activation = activation or ("gelu_tanh" if tanh_form else "gelu")
        if self.activation not in ops.stream.ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not one of {sorted(ops.stream.ACTIVATIONS)}")
        self.up = self.down = None

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, i = self.prefix, self.hidden_size, self.intermediate_size
        return [TensorSpec(p + "up", (i, d)), TensorSpec(p + "down", (d, i))]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.up, self.down = tensors[self.prefix + "up"], tensors[self.prefix + "down"]

    def inner(self, h: torch.Tensor) -> torch.Tensor:
        """act(up h): the squared ReLU inside the product's epilogue where the tensor-core GEMM runs it."""
        if self.activation == "relu2":
            fused = ops.linear_relu2(h, self.up)
            if fused is not None:
                return fused
        return ops.activation(ops.linear(h, self.up), self.activation)

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext) -> torch.Tensor:
        inner = self.inner(h)
        # without a residual (a block that sums in float32 itself) the product stays float32
        return ops.linear(inner, self.down, residual, out_dtype=torch.float32 if residual is None else None)

    def forward_for_stream(self, h: torch.Tensor, ctx: StepContext):
        """ff(h) for a block that adds it to a float32 stream and norms the sum at once: float32, or
        the down projection's partial sums for that norm to add up (`ops.linear_for_stream`)."""
        return ops.linear_for_stream(self.inner(h), self.down)


class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, prefix: str, experts: int, top: int, expert_ff: int, limit: float = 0.0,
                 groups: int = 1, group_top: int = 2, keep: int = 1, scale: float = 1.0, slope: float = 1.0,
                 shift: float = 0.0, score: str = "sigmoid", renormalise: bool = True, shared_ff: int | None = None,
                 shared_limit: float | None = None, shared_gated: bool = True, identity: int = 0,
                 choice_offsets: bool = False):  # fmt: skip
        # `identity`: that many further router outputs are experts without tensors whose output is their
        # input; `choice_offsets`: a learned vector (`correction`) joins the scores when the experts are
        # chosen and stays out of their weights
        self.identity, self.choice_offsets = int(identity), bool(choice_offsets)
        if self.identity and groups != 1:
            raise ValueError("identity experts belong to no group of experts")
        if experts % groups or not 1 <= keep <= groups or not 1 <= top <= (experts + self.identity) // groups * keep:
            raise ValueError(f"{experts} experts in {groups} groups, {keep} kept, cannot give {top} choices")
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"score {score!r} is neither 'sigmoid' nor 'softmax'")
        self.hidden_size, self.prefix = hidden_size, prefix
        self.experts, self.top, self.expert_ff, self.limit = experts, top, expert_ff, float(limit)
        self.groups, self.group_top, self.keep, self.scale = groups, group_top, keep, float(scale)
        self.slope, self.shift, self.score, self.renormalise = float(slope), float(shift), score, renormalise
        self.shared_ff, self.shared_gated = shared_ff, shared_gated and shared_ff is not None
        self.shared_limit = float(limit if shared_limit is None else shared_limit)
        self.router = self.gate = self.up = self.down = self.shared_gate_up = self.shared_down = None

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, f = self.prefix, self.hidden_size, self.expert_ff
        specs = []
        for e in range(self.experts):
            specs += [TensorSpec(f"{p}e{e}.gate", (f, d)), TensorSpec(f"{p}e{e}.up", (f, d)), TensorSpec(f"{p}e{e}.down", (d, f))]
        specs.append(TensorSpec(p + "router", (self.experts + self.identity, d)))
        if self.choice_offsets:
            specs.append(TensorSpec(p + "correction", (self.experts + self.identity,), kind="gain", init="normal"))
        if self.shared_ff is not None:
            s = self.shared_ff
            specs += [TensorSpec(p + "shared.gate", (s, d)), TensorSpec(p + "shared.up", (s, d)), TensorSpec(p + "shared.down", (d, s))]
            if self.shared_gated:
                specs.append(TensorSpec(p + "shared.sg", (1, d)))
        return specs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p, E = self.prefix, self.experts
        self.gate = torch.stack([tensors[f"{p}e{e}.gate"] for e in range(E)]).contiguous()  # [E, F, d]
        self.up = torch.stack([tensors[f"{p}e{e}.up"] for e in range(E)]).contiguous()
        self.down = torch.stack([tensors[f"{p}e{e}.down"] for e in range(E)]).contiguous()  # [E, d, F]
        rows = [tensors[p + "router"]]
        if self.shared_ff is not None:
            if self.shared_gated:
                rows.append(tensors[p + "shared.sg"])  # the shared expert's gate rides in the router's product
            self.shared_gate_up = torch.cat([tensors[p + "shared.gate"], tensors[p + "shared.up"]]).contiguous()
            self.shared_down = tensors[p + "shared.down"]
        self.router = torch.cat(rows).contiguous()
        self.offsets = tensors[p + "correction"].contiguous() if self.choice_offsets else None

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext) -> torch.Tensor:
        E, routed = self.experts, self.experts + self.identity
        z = ops.linear(h, self.router, out_dtype=torch.float32)
        ids, weights, shared_gate = ops.route(
            z, experts=routed, top=self.top, groups=self.groups, group_top=self.group_top, keep=self.keep, scale=self.scale,
            gate_col=routed if self.shared_gated else None, softmax=self.score == "softmax", renormalise=self.renormalise,
            bias=self.offsets,
        )  # fmt: skip
        # (the identity experts' pairs are sorted behind the last expert's rows, where no product looks)
        offsets, row_token, pair_row = ops.group_by_expert(ids, routed)
        hidden = ops.experts_glu(h, row_token, offsets, self.gate, self.up, self.limit, self.slope, self.shift)
        y = ops.experts_down(hidden, offsets, self.down)
        shared = None
        if self.shared_ff is not None:
            inner = ops.clamped_glu(ops.linear(h, self.shared_gate_up), self.shared_limit, self.slope, self.shift)
            shared = ops.linear(inner, self.shared_down, out_dtype=torch.float32 if residual is None else None)
        out = ops.combine(y, pair_row, weights, shared, shared_gate, identity=(ids, h, E) if self.identity else None)
        if residual is None:
            return out
        return residual + out.to(residual.dtype)


class NoFeedForward(FeedForward):
    """The feed-forward of a layer that has none."""

    absent = True

    def __init__(self, hidden_size: int, prefix: str):
        pass

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext) -> torch.Tensor:
        raise RuntimeError("this layer has no feed-forward")


register_part("feed_forward", "gelu_mlp", GeluMLP)
register_part("feed_forward", "activation_mlp", GeluMLP)
register_part("feed_forward", "routed_experts", RoutedExperts)
register_part("feed_forward", "none", NoFeedForward)
