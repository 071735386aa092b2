"""What surrounds a selective state-space recurrence (csrc/ssm.cu): the causal convolution per
channel with the step sizes, the convolution's per-request state, and the gated norm in parts of
the row. The recurrence itself is `linear_recurrence` with shared q and k."""

from __future__ import annotations

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream


def _f32(t: torch.Tensor | None, shape: tuple, name: str) -> None:
    if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous()):
        raise KernelLibraryError(f"{name} must be contiguous float32 {list(shape)}, got {t.dtype} {tuple(t.shape)}")


def conv_steps(proj: torch.Tensor, conv_off: int, dt_off: int, taps: torch.Tensor, bias: torch.Tensor,
               conv_state: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, state_slots: torch.Tensor,
               req_q_start: torch.Tensor, num_requests: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:  # fmt: skip
    """From a projection [T, columns] in the compute dtype, per request in token order:

    conv: C = taps.shape[0] channels from column conv_off through a causal convolution of K taps
    (the last tap is the current token's), plus bias, then SiLU; what lies before a portion's first
    token is read from `conv_state` [slots, K - 1, C] (float32; zeros for a new request), which this
    call does not change (`conv_state_update` does). Returns it as [T, C] in the compute dtype.

    steps: H = dt_bias.shape[0] columns from dt_off: dt = softplus(z + dt_bias); returns the
    per-token decay exp(-exp(a_log) dt) and input weight dt, float32 [T, H] each."""
    require_cuda(proj, taps, bias, conv_state, dt_bias, a_log, state_slots, req_q_start)
    if proj.dim() != 2 or not proj.is_contiguous():
        raise KernelLibraryError("conv_steps: proj must be a contiguous [tokens, columns] tensor")
    T = proj.shape[0]
    C, K = taps.shape
    H = dt_bias.shape[0]
    _f32(taps, (C, K), "taps")
    _f32(bias, (C,), "bias")
    _f32(conv_state, (conv_state.shape[0], max(K - 1, 0), C), "conv_state")
    _f32(dt_bias, (H,), "dt_bias")
    _f32(a_log, (H,), "a_log")
    if conv_off + C > proj.shape[1] or dt_off + H > proj.shape[1]:
        raise KernelLibraryError("conv_steps: the column ranges lie outside proj")
    for t in (state_slots, req_q_start):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelLibraryError("conv_steps: index tensors must be contiguous int32")
    out = torch.empty(T, C, device=proj.device, dtype=proj.dtype)
    decay = torch.empty(T, H, device=proj.device, dtype=torch.float32)
    weight = torch.empty_like(decay)
    check(lib().asb_conv_steps(ptr(out), ptr(decay), ptr(weight), ptr(proj), proj.shape[1], conv_off, dt_off, ptr(taps),
                               ptr(bias), ptr(conv_state), ptr(dt_bias), ptr(a_log), ptr(state_slots), ptr(req_q_start),
                               T, num_requests, C, K, H, dtype_code(proj), stream()))  # fmt: skip
    return out, decay, weight


def conv_state_update(conv_state: torch.Tensor, proj: torch.Tensor, conv_off: int, state_slots: torch.Tensor,
                      req_q_start: torch.Tensor, num_requests: int) -> None:  # fmt: skip
    """Leave in `conv_state` [slots, K - 1, C] the last K - 1 convolution inputs of every request of
    the step (columns from conv_off of proj); a portion shorter than K - 1 shifts what was held."""
    require_cuda(conv_state, proj, state_slots, req_q_start)
    _, taps_held, C = conv_state.shape
    if conv_state.dtype != torch.float32 or not conv_state.is_contiguous() or conv_off + C > proj.shape[1]:
        raise KernelLibraryError("conv_state_update: a contiguous float32 state whose channels lie inside proj")
    check(lib().asb_conv_state_update(ptr(conv_state), ptr(proj), proj.shape[1], conv_off, ptr(state_slots), ptr(req_q_start),
                                      num_requests, C, taps_held + 1, dtype_code(proj), stream()))  # fmt: skip


def gate_group_norm(y: torch.Tensor, x: torch.Tensor | None, z: torch.Tensor, skip: torch.Tensor | None, gain: torch.Tensor,
                    parts: int, head_width: int, eps: float) -> torch.Tensor:  # fmt: skip
    """v = (y + skip_h x) silu(z) (the skip term where `skip` [heads] is given), RMS-normed in `parts`
    equal parts of the row, each by its own root mean square, times gain. y: float32 [T, width]; x and
    z: [T, width] in the compute dtype, rows may be strided (column ranges of a wider tensor).
    Returns [T, width] in the compute dtype."""
    require_cuda(y, x, z, skip, gain)
    T, width = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous() or z.shape != y.shape or z.stride(1) != 1:
        raise KernelLibraryError("gate_group_norm: y contiguous float32 [T, width], z of its shape with unit column stride")
    if skip is not None:
        _f32(skip, (width // head_width,), "skip")
        if x is None or x.shape != y.shape or x.stride(1) != 1 or x.dtype != z.dtype:
            raise KernelLibraryError("gate_group_norm: the skip term needs x of y's shape in z's dtype")
    _f32(gain, (width,), "gain")
    out = torch.empty(T, width, device=y.device, dtype=z.dtype)
    check(lib().asb_gate_group_norm(ptr(out), ptr(y), ptr(x) if skip is not None else None, x.stride(0) if skip is not None else 0,
                                    ptr(z), z.stride(0), ptr(skip), ptr(gain), T, width, parts, head_width, float(eps),
                                    dtype_code(z), stream()))  # fmt: skip
    return out
