"""RMSNorm: gain * x / sqrt(mean(x^2) + eps), float32 inside, one rounding
(atomserve/model.py:125-139)."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import Norm, register_part
from atomserve_b200.parts.spec import TensorSpec


class RMSNorm(Norm):
    def __init__(self, hidden_size: int, prefix: str, eps: float, width: int | None = None, tensor: str | None = None):
        self.width = width or hidden_size
        self.eps = float(eps)
        self.name = tensor or prefix + "weight"
        self.gain: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.width,), kind="gain", init="gain")]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.gain = tensors[self.name]

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        return ops.rms_norm(x, self.gain, self.eps, rows)

    def after_linear(self, x: torch.Tensor, weight: torch.Tensor,
                     residual: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
        """(s, forward(s)) for s = x . weight^T + residual. Where the product runs with partial
        sums (few tokens), one kernel adds them up, adds the residual and normalises; the results
        are the same bits either way."""
        if ops.partial_add_rms_norm_fusable(self.width) and weight.shape[0] == self.width:
            product = ops.linear_partial(x, weight)
            if product is not None:
                return ops.partial_add_rms_norm(product, residual, self.gain, self.eps)
        total = ops.linear(x, weight, residual)
        return total, self.forward(total)


class ScaledRMSNorm(RMSNorm):
    """An RMS norm that also carries `mult`, the factor by which its block multiplies what the
    sublayers give before adding it to the stream (blocks that sum their sublayers themselves)."""

    def __init__(self, hidden_size: int, prefix: str, eps: float, mult: float = 1.0, width: int | None = None,
                 tensor: str | None = None):  # fmt: skip
        super().__init__(hidden_size, prefix, eps, width, tensor)
        self.mult = float(mult)


class StreamRMSNorm(RMSNorm):
    """RMSNorm of a residual stream that is kept in float32 whatever the compute dtype, for
    blocks whose norm follows the sum: `add_forward(x, y)` is norm(alpha x + y), returned both as
    the new float32 stream and in the compute dtype (what the next products read); `forward` is
    the plain norm of (rows of) the stream in the compute dtype, as a final norm before the head."""

    def __init__(self, hidden_size: int, prefix: str, eps: float, alpha: float = 1.0, width: int | None = None,
                 tensor: str | None = None):  # fmt: skip
        super().__init__(hidden_size, prefix, eps, width, tensor)
        self.alpha = float(alpha)
        self.dtype = torch.float32

    def bind_dtype(self, dtype: torch.dtype) -> None:
        self.dtype = dtype

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        return ops.scaled_add_rms_norm(x, None, 1.0, self.gain, self.eps, self.dtype, rows, want_stream=False)[1]

    def add_forward(self, x: torch.Tensor, y: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        return ops.scaled_add_rms_norm(x, y, self.alpha, self.gain, self.eps, self.dtype)


class OutputNorm(Norm):
    """The norm of a block that norms each sublayer's output and adds it to a float32 stream:
    `add_forward(x, y)` is x + mult * N(y) * gain * scale, returned as the new stream and in the
    compute dtype. N is the centred norm (y - mean) / sqrt(var + eps), gain only, no bias, or with
    `centred=False` the RMS norm; `scale_tensor` names a per-channel layer scale, if the layer has
    one. `forward` is N(x) * gain of (rows of) the stream in the compute dtype, as a final norm."""

    def __init__(self, hidden_size: int, prefix: str, eps: float, mult: float = 1.0, centred: bool = True,
                 tensor: str | None = None, scale_tensor: str | None = None):  # fmt: skip
        self.width, self.eps, self.mult, self.centred = hidden_size, float(eps), float(mult), bool(centred)
        self.name, self.scale_name = tensor or prefix + "weight", scale_tensor
        self.gain = self.scale = None
        self.dtype = torch.float32

    def tensor_specs(self) -> list[TensorSpec]:
        specs = [TensorSpec(self.name, (self.width,), kind="gain", init="gain")]
        if self.scale_name:
            specs.append(TensorSpec(self.scale_name, (self.width,), kind="gain", init="gain"))
        return specs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.gain = tensors[self.name]
        self.scale = tensors[self.scale_name] if self.scale_name else None

    def bind_dtype(self, dtype: torch.dtype) -> None:
        self.dtype = dtype

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        return ops.residual_out_norm(None, x, self.gain, self.eps, self.dtype, centred=self.centred, rows=rows, want_stream=False)[1]

    def add_forward(self, x: torch.Tensor, y: torch.Tensor, halves=None) -> tuple[torch.Tensor, torch.Tensor]:
        """`halves=(b, gain_a, gain_b)`: the sublayer's output is (R(y) gain_a + R(b) gain_b) / 2 with
        R the unit-RMS norm (two mixers side by side), formed in the same kernel."""
        return ops.residual_out_norm(x, y, self.gain, self.eps, self.dtype, mult=self.mult, scale=self.scale,
                                     centred=self.centred, halves=halves)  # fmt: skip


class SandwichNorm(Norm):
    """The two norms around one sublayer of a block that norms a sublayer's input and its output
    over a float32 stream, x <- x + N_out(f(N_in(x))), both RMS norms with a gain: `forward` is
    N_in of (rows of) the stream in the compute dtype; `add_forward(x, y, then, bias)` is the new
    stream x + N_out(y + bias) and, where `then` (the norm whose input comes next) is given, that
    norm's N_in of it in the compute dtype, from one kernel. `tensor` and `out_tensor` name the
    two gains."""

    def __init__(self, hidden_size: int, prefix: str, eps: float, tensor: str | None = None, out_tensor: str | None = None):
        self.width, self.eps = hidden_size, float(eps)
        self.name, self.out_name = tensor or prefix + "weight", out_tensor or prefix + "out.weight"
        self.gain = self.out_gain = None
        self.dtype = torch.float32

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.width,), kind="gain", init="gain"),
                TensorSpec(self.out_name, (self.width,), kind="gain", init="gain")]  # fmt: skip

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.gain, self.out_gain = tensors[self.name], tensors[self.out_name]

    def bind_dtype(self, dtype: torch.dtype) -> None:
        self.dtype = dtype

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        return ops.scaled_add_rms_norm(x, None, 1.0, self.gain, self.eps, self.dtype, rows, want_stream=False)[1]

    def add_forward(self, x: torch.Tensor, y, then: Norm | None = None, bias: torch.Tensor | None = None):
        gain_next = getattr(then, "gain", None) if then is not None else None
        if then is not None and (gain_next is None or not hasattr(then, "eps")):
            stream, _ = ops.add_normed(x, y, self.out_gain, self.eps, None, 0.0, self.dtype, bias)
            return stream, then.forward(stream)
        return ops.add_normed(x, y, self.out_gain, self.eps, gain_next, then.eps if then is not None else 0.0, self.dtype, bias)


class NoNorm(Norm):
    """The norm of a sublayer that a layer does not have."""

    def __init__(self, hidden_size: int, prefix: str):
        pass

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        raise RuntimeError("this layer has no such norm")


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "scaled_rms_norm", ScaledRMSNorm)
register_part("norm", "stream_rms_norm", StreamRMSNorm)
register_part("norm", "output_norm", OutputNorm)
register_part("norm", "sandwich_norm", SandwichNorm)
register_part("norm", "none", NoNorm)
