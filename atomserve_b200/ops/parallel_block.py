"""Operations of layers whose mixer and feed-forward read the same float32 stream and are added
together, of a token embedding with a hashed table of token pairs beside it, and of a product over
two streams: the Python faces of csrc/parallel_block.cu."""

from __future__ import annotations

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream


def _rows32(t: torch.Tensor | None, name: str, shape: tuple) -> None:
    if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous()):
        raise KernelLibraryError(f"{name} must be contiguous float32 {list(shape)}, got {t.dtype} {tuple(t.shape)}")


def residual_dual_norm(x: torch.Tensor | None, y1: torch.Tensor | None, y2: torch.Tensor | None, mult: float,
                       gain1: torch.Tensor | None, gain2: torch.Tensor | None, eps: float, dtype: torch.dtype, *,
                       bias: torch.Tensor | None = None,
                       want_stream: bool = True) -> tuple[torch.Tensor | None, torch.Tensor | None, torch.Tensor | None]:  # fmt: skip
    """s = x + mult (y1 + y2) + bias, every term optional (float32 [n, width]; bias [width]), and
    its two norms N(s) gain1, N(s) gain2 in `dtype`, N(s) = s / sqrt(mean(s^2) + eps). Returns
    (s or None, first norm or None, second norm or None)."""
    first = next((t for t in (x, y1, y2) if t is not None), None)
    if first is None:
        raise KernelLibraryError("residual_dual_norm: nothing to add")
    require_cuda(x, y1, y2, bias, gain1, gain2)
    n, width = first.shape
    for t, name in ((x, "x"), (y1, "y1"), (y2, "y2")):
        _rows32(t, name, (n, width))
    for t, name in ((bias, "bias"), (gain1, "gain1"), (gain2, "gain2")):
        _rows32(t, name, (width,))
    out32 = torch.empty(n, width, device=first.device, dtype=torch.float32) if want_stream else None
    out1 = torch.empty(n, width, device=first.device, dtype=dtype) if gain1 is not None else None
    out2 = torch.empty(n, width, device=first.device, dtype=dtype) if gain2 is not None else None
    code = dtype_code(out1 if out1 is not None else out2) if (out1 is not None or out2 is not None) else 0
    check(lib().asb_residual_dual_norm(ptr(out32), ptr(out1), ptr(out2), ptr(x), ptr(y1), ptr(y2), ptr(bias), ptr(gain1),
                                       ptr(gain2), n, width, float(mult), float(eps), code, stream()))  # fmt: skip
    return out32, out1, out2


def pair_embedding(ids: torch.Tensor, positions: torch.Tensor, req_q_start: torch.Tensor, state_slots: torch.Tensor,
                   last_id: torch.Tensor, table: torch.Tensor, pairs: torch.Tensor, mul_prev: int, mul_cur: int,
                   status: torch.Tensor) -> torch.Tensor:  # fmt: skip
    """float32 out[t] = table[ids[t]] + pairs[(previous id * mul_prev + ids[t] * mul_cur) mod buckets],
    `pairs` having buckets + 1 rows, the last one for a token at position 0. The id before a
    request's first token of the step is last_id[slot] - 1 (int32 per state slot), which is then
    set to the request's last id of the step plus one."""
    require_cuda(ids, positions, req_q_start, state_slots, last_id, table, pairs, status)
    for t in (ids, positions, req_q_start, state_slots, last_id):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelLibraryError("pair_embedding: index tensors must be contiguous int32")
    if table.dim() != 2 or pairs.dim() != 2 or pairs.shape[1] != table.shape[1] or pairs.dtype != table.dtype or pairs.shape[0] < 2:
        raise KernelLibraryError("pair_embedding: the two tables must share width and dtype")
    if not table.is_contiguous() or not pairs.is_contiguous():
        raise KernelLibraryError("pair_embedding: tables must be contiguous")
    out = torch.empty(ids.shape[0], table.shape[1], device=table.device, dtype=torch.float32)
    check(lib().asb_pair_embedding(ptr(out), ptr(table), ptr(pairs), ptr(ids), ptr(positions), ptr(req_q_start),
                                   ptr(state_slots), ptr(last_id), ids.shape[0], state_slots.shape[0], table.shape[1],
                                   table.shape[0], pairs.shape[0] - 1, int(mul_prev), int(mul_cur), dtype_code(table),
                                   ptr(status), stream()))  # fmt: skip
    return out


def concat_cast(a: torch.Tensor, b: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """[a ; b] per row in `dtype`, a and b float32 [n, width]."""
    require_cuda(a, b)
    _rows32(a, "a", tuple(a.shape))
    _rows32(b, "b", tuple(a.shape))
    out = torch.empty(a.shape[0], 2 * a.shape[1], device=a.device, dtype=dtype)
    check(lib().asb_concat_cast(ptr(out), ptr(a), ptr(b), a.shape[0], a.shape[1], dtype_code(out), stream()))
    return out
