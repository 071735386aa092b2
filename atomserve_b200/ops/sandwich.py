"""Operations of blocks that norm a sublayer's input and its output over a float32 stream, a gated
feed-forward's activation with biases, and the soft cap of logits (csrc/sandwich_norm.cu)."""

from __future__ import annotations

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream
from atomserve_b200.ops.linear import GLU_ACTIVATIONS, PartialSums


def add_normed(x: torch.Tensor, y: torch.Tensor | PartialSums, gain_out: torch.Tensor, eps_out: float,
               gain_next: torch.Tensor | None, eps_next: float, dtype: torch.dtype,
               bias: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor | None]:  # fmt: skip
    """s = x + N(y + bias) gain_out, N(v) = v / sqrt(mean(v^2) + eps); and with `gain_next`,
    N(s) gain_next in `dtype`: the next sublayer's input. x: float32 [n, width]; y: float32 or
    bfloat16 of that shape, or the partial sums of a product (`linear_for_stream`), which the kernel
    adds up itself. Returns (s float32, the normed copy or None)."""
    n, width = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelLibraryError("add_normed: x must be a contiguous float32 [rows, width] tensor")
    for t, name in ((gain_out, "gain_out"), (gain_next, "gain_next"), (bias, "bias")):
        if t is not None and (t.dtype != torch.float32 or t.shape != (width,) or not t.is_contiguous()):
            raise KernelLibraryError(f"add_normed: {name} must be contiguous float32 [{width}]")
    out32 = torch.empty_like(x)
    out_c = torch.empty(n, width, device=x.device, dtype=dtype) if gain_next is not None else None
    if isinstance(y, PartialSums):
        require_cuda(x, gain_out, gain_next, bias)
        if dtype != torch.bfloat16 or (y.tokens, y.columns) != (n, width):
            raise KernelLibraryError("add_normed: partial sums are of bfloat16 products of the stream's shape")
        check(lib().asb_partial_add_normed(ptr(out32), ptr(out_c), ptr(y.workspace), *y.layout(), ptr(x), ptr(bias),
                                           ptr(gain_out), ptr(gain_next), n, width, float(eps_out), float(eps_next), stream()))  # fmt: skip
        return out32, out_c
    require_cuda(x, y, gain_out, gain_next, bias)
    if y.shape != x.shape or not y.is_contiguous() or y.dtype not in (torch.float32, torch.bfloat16):
        raise KernelLibraryError("add_normed: y must match x in shape, contiguous, float32 or bfloat16")
    check(lib().asb_add_normed(ptr(out32), ptr(out_c), ptr(x), ptr(y), dtype_code(y), ptr(bias), ptr(gain_out), ptr(gain_next),
                               n, width, float(eps_out), float(eps_next), dtype_code(out_c) if out_c is not None else 0,
                               stream()))  # fmt: skip
    return out32, out_c


def bias_glu(gate_up: torch.Tensor, bias: torch.Tensor | None, activation: str) -> torch.Tensor:
    """[T, 2F] (gate columns first) -> act(gate + bias[:F]) * (up + bias[F:]); act "silu",
    "gelu_tanh" or "gelu"; float32 inside."""
    require_cuda(gate_up, bias)
    if activation not in GLU_ACTIVATIONS:
        raise KernelLibraryError(f"bias_glu: activation {activation!r} is not one of {sorted(GLU_ACTIVATIONS)}")
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise KernelLibraryError("bias_glu takes a contiguous [tokens, 2 * intermediate] tensor")
    inter = gate_up.shape[1] // 2
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (2 * inter,) or not bias.is_contiguous()):
        raise KernelLibraryError(f"bias_glu: bias must be contiguous float32 [{2 * inter}]")
    out = torch.empty(gate_up.shape[0], inter, device=gate_up.device, dtype=gate_up.dtype)
    check(lib().asb_bias_glu(ptr(out), ptr(gate_up), ptr(bias), gate_up.shape[0], inter, GLU_ACTIVATIONS[activation],
                             dtype_code(gate_up), stream()))  # fmt: skip
    return out


def softcap_(values: torch.Tensor, cap: float) -> torch.Tensor:
    """values <- cap tanh(values / cap), in place; float32."""
    require_cuda(values)
    if values.dtype != torch.float32 or not values.is_contiguous():
        raise KernelLibraryError("softcap_ takes a contiguous float32 tensor")
    check(lib().asb_softcap(ptr(values), values.numel(), float(cap), stream()))
    return values
