"""Routed experts (csrc/moe.cu): selection from router logits, grouping of the step's
(token, expert) pairs by expert, the experts' products over the grouped rows, and the weighted
sum back per token."""

from __future__ import annotations

import os

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream


# Which kernels multiply the experts in bfloat16: "mma" (tensor cores, csrc/moe_mma.cu; the default
# where K is a multiple of 8) or "simt" (the CUDA-core kernels that float32 always runs).
EXPERT_KERNELS = os.environ.get("ATOMSERVE_B200_EXPERTS", "mma")


def _tensor_cores(x: torch.Tensor, *weights: torch.Tensor) -> bool:
    return (EXPERT_KERNELS == "mma" and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and all(t.data_ptr() % 16 == 0 for t in (x, *weights)))  # fmt: skip


def route(z: torch.Tensor, *, experts: int, top: int, groups: int = 1, group_top: int = 2, keep: int = 1,
          scale: float = 1.0, gate_col: int | None = None, softmax: bool = False,
          renormalise: bool = True, bias: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor | None]:  # fmt: skip
    """z: float32 [T, >= experts] router logits. Returns (ids int32 [T, top], weights float32
    [T, top], sigmoid(z[:, gate_col]) float32 [T] or None). `bias` (float32 [experts]) is added to
    the scores for the final choice only; the weights are made of the scores themselves."""
    require_cuda(z, bias)
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (experts,) or not bias.is_contiguous()):
        raise KernelLibraryError(f"route: bias must be contiguous float32 [{experts}]")
    if z.dtype != torch.float32 or z.dim() != 2 or z.stride(1) != 1 or z.shape[1] < experts:
        raise KernelLibraryError("route: z must be float32 [tokens, >= experts] with unit column stride")
    T = z.shape[0]
    ids = torch.empty(T, top, device=z.device, dtype=torch.int32)
    weights = torch.empty(T, top, device=z.device, dtype=torch.float32)
    shared = torch.empty(T, device=z.device, dtype=torch.float32) if gate_col is not None else None
    check(lib().asb_moe_route_biased(ptr(z), z.stride(0), T, experts, groups, group_top, keep, top,
                                     -1 if gate_col is None else gate_col, int(softmax), int(renormalise), float(scale),
                                     ptr(bias), ptr(ids), ptr(weights), ptr(shared), stream()))  # fmt: skip
    return ids, weights, shared


def group_by_expert(ids: torch.Tensor, experts: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(offsets int32 [E + 1], row_token int32 [T * top], pair_row int32 [T, top]): the pairs
    sorted by expert, expert e owning sorted rows offsets[e] : offsets[e + 1]."""
    require_cuda(ids)
    T, top = ids.shape
    offsets = torch.empty(experts + 1, device=ids.device, dtype=torch.int32)
    row_token = torch.empty(T * top, device=ids.device, dtype=torch.int32)
    pair_row = torch.empty(T, top, device=ids.device, dtype=torch.int32)
    check(lib().asb_moe_group(ptr(ids), T, top, experts, ptr(offsets), ptr(row_token), ptr(pair_row), stream()))
    return offsets, row_token, pair_row


def experts_glu(x: torch.Tensor, row_token: torch.Tensor, offsets: torch.Tensor, gate: torch.Tensor, up: torch.Tensor,
                limit: float, slope: float, shift: float) -> torch.Tensor:  # fmt: skip
    """hidden [pairs, F]: for the sorted rows of expert e, act(x[token] . gate[e]^T, x[token] . up[e]^T)."""
    require_cuda(x, row_token, offsets, gate, up)
    E, F, K = gate.shape
    if up.shape != gate.shape or x.shape[1] != K or x.dtype != gate.dtype or not (x.is_contiguous() and gate.is_contiguous() and up.is_contiguous()):
        raise KernelLibraryError("experts_glu: x [T, K] against gate and up [E, F, K] of one dtype, contiguous")
    pairs = row_token.shape[0]
    hidden = torch.empty(pairs, F, device=x.device, dtype=x.dtype)
    if _tensor_cores(x, gate, up):
        check(lib().asb_moe_glu_mma(ptr(hidden), ptr(x), ptr(row_token), ptr(offsets), ptr(gate), ptr(up), pairs, E, F, K,
                                    float(limit), float(slope), float(shift), stream()))  # fmt: skip
        return hidden
    check(lib().asb_moe_glu(ptr(hidden), ptr(x), ptr(row_token), ptr(offsets), ptr(gate), ptr(up), pairs, E, F, K,
                            float(limit), float(slope), float(shift), dtype_code(x), stream()))  # fmt: skip
    return hidden


def experts_down(hidden: torch.Tensor, offsets: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """y float32 [pairs, N]: hidden[row] . down[e]^T for the sorted rows of expert e."""
    require_cuda(hidden, offsets, down)
    E, N, F = down.shape
    if hidden.shape[1] != F or hidden.dtype != down.dtype or not (hidden.is_contiguous() and down.is_contiguous()):
        raise KernelLibraryError("experts_down: hidden [pairs, F] against down [E, N, F] of one dtype, contiguous")
    y = torch.empty(hidden.shape[0], N, device=hidden.device, dtype=torch.float32)
    if _tensor_cores(hidden, down):
        check(lib().asb_moe_down_mma(ptr(y), ptr(hidden), ptr(offsets), ptr(down), hidden.shape[0], E, N, F, stream()))
        return y
    check(lib().asb_moe_down(ptr(y), ptr(hidden), ptr(offsets), ptr(down), hidden.shape[0], E, N, F, dtype_code(hidden), stream()))
    return y


def combine(y: torch.Tensor, pair_row: torch.Tensor, weights: torch.Tensor, shared: torch.Tensor | None = None,
            shared_gate: torch.Tensor | None = None, *, identity: tuple[torch.Tensor, torch.Tensor, int] | None = None) -> torch.Tensor:  # fmt: skip
    """float32 out[t] = sum_k weights[t, k] y[pair_row[t, k]] (+ shared_gate[t] * shared[t]; without a
    gate, + shared[t]). `identity=(ids, x, experts)`: a choice ids[t, k] >= experts is an identity
    expert, whose output is the token's own input row x[t] instead of a row of y."""
    require_cuda(y, pair_row, weights, shared, shared_gate)
    ids, x, experts = identity if identity is not None else (None, None, 0)
    if identity is not None:
        require_cuda(ids, x)
        if ids.shape != pair_row.shape or ids.dtype != torch.int32 or x.shape != (pair_row.shape[0], y.shape[1]) or not x.is_contiguous():
            raise KernelLibraryError("combine: identity experts need ids [tokens, top] and the input rows [tokens, width]")
    T, top = pair_row.shape
    N = y.shape[1]
    if shared is not None and (shared.shape != (T, N) or not shared.is_contiguous()):
        raise KernelLibraryError("combine: shared must be a contiguous [tokens, width] tensor")
    out = torch.empty(T, N, device=y.device, dtype=torch.float32)
    check(lib().asb_moe_combine_identity(ptr(out), ptr(y), ptr(pair_row), ptr(weights), ptr(shared), ptr(shared_gate), T, top, N,
                                         dtype_code(shared) if shared is not None else 0, ptr(ids), ptr(x),
                                         dtype_code(x) if x is not None else 0, int(experts), stream()))  # fmt: skip
    return out
