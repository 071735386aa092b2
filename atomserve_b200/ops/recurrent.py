"""Linear attention over per-request state, S <- a S + b k v^T, o = S^T q: with a fixed decay per
head ("lightning attention", retention) or a decay and an input weight per token (gated matrix
memories), optionally with a normaliser and a rotation of q and k (csrc/lightning.cu)."""

from __future__ import annotations

import dataclasses

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream


SEGMENT_TOKENS = 64  # tokens of a segment when a long portion is cut to run side by side
SEGMENT_FROM = 256  # a request bringing at least this many tokens is cut


@dataclasses.dataclass
class Segments:
    """A step's requests cut into segments of consecutive rows: `bounds` int32 [S + 1] (rows),
    `req_start` int32 [R + 1] (the segments of each request), `index` int32 [S] = 0..S-1."""

    bounds: torch.Tensor
    req_start: torch.Tensor
    index: torch.Tensor
    count: int


def plan_segments(q_lens: list[int], device: torch.device) -> Segments | None:
    """The segments of a step whose requests bring `q_lens` tokens, or None when no request is
    long enough to be worth cutting (decode steps, short portions)."""
    if not q_lens or max(q_lens) < SEGMENT_FROM:
        return None
    bounds, req_start, row = [0], [0], 0
    for n in q_lens:
        pieces = -(-n // SEGMENT_TOKENS) if n >= SEGMENT_FROM else 1
        for i in range(pieces):
            bounds.append(row + min(n, (i + 1) * SEGMENT_TOKENS) if n >= SEGMENT_FROM else row + n)
        row += n
        req_start.append(len(bounds) - 1)
    count = len(bounds) - 1
    packed = torch.tensor(bounds + req_start + list(range(count)), dtype=torch.int32).to(device, non_blocking=True)
    a, b = len(bounds), len(bounds) + len(req_start)
    return Segments(packed[:a], packed[a:b], packed[b:], count)


def lightning_attention(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, state: torch.Tensor,
                        state_slots: torch.Tensor, req_q_start: torch.Tensor, decay: torch.Tensor,
                        num_requests: int, activation: bool = True, segments: Segments | None = None) -> torch.Tensor:  # fmt: skip
    """S <- decay_h S + k v^T, o = S^T q for every new token of every request, in order; the
    state [slots, H, D, V] (float32) is read and left updated in each request's slot.

    proj: [T, W] in the compute dtype, holding q (H * D columns from q_off), k (from k_off) and v
    (H * V columns from v_off), head by head; `activation`: SiLU on all three. Returns float32
    [T, H * V]. With `segments` (`plan_segments`) long portions run as segments side by side: each
    from a zero state, then a walk over each request's segments that hands every segment the
    state it starts from, then that state's share added to the segment's tokens."""
    require_cuda(proj, state, state_slots, req_q_start, decay)
    if proj.dim() != 2 or not proj.is_contiguous():
        raise KernelLibraryError("lightning_attention: proj must be a contiguous [tokens, columns] tensor")
    if state.dtype != torch.float32 or state.dim() != 4 or not state.is_contiguous():
        raise KernelLibraryError("lightning_attention: state must be contiguous float32 [slots, H, D, V]")
    _, H, D, V = state.shape
    if decay.dtype != torch.float32 or decay.shape != (H,):
        raise KernelLibraryError(f"lightning_attention: decay must be float32 [{H}]")
    for t in (state_slots, req_q_start):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelLibraryError("lightning_attention: index tensors must be contiguous int32")
    if max(q_off, k_off) + H * D > proj.shape[1] or v_off + H * V > proj.shape[1]:
        raise KernelLibraryError("lightning_attention: the column ranges lie outside proj")
    out = torch.empty(proj.shape[0], H * V, device=proj.device, dtype=torch.float32)
    if segments is None:
        check(lib().asb_lightning_attention(ptr(out), ptr(proj), proj.shape[1], q_off, k_off, v_off, ptr(state),
                                            ptr(state_slots), ptr(req_q_start), ptr(decay), num_requests, H, D, V,
                                            int(activation), 0, dtype_code(proj), stream()))  # fmt: skip
        return out
    local = torch.empty(segments.count, H, D, V, device=proj.device, dtype=torch.float32)
    for mode in (1, 2):
        if mode == 2:
            check(lib().asb_lightning_scan(ptr(local), ptr(state), ptr(state_slots), ptr(segments.req_start),
                                           ptr(segments.bounds), ptr(decay), num_requests, H, D, V, stream()))  # fmt: skip
        check(lib().asb_lightning_attention(ptr(out), ptr(proj), proj.shape[1], q_off, k_off, v_off, ptr(local),
                                            ptr(segments.index), ptr(segments.bounds), ptr(decay), segments.count, H, D, V,
                                            int(activation), mode, dtype_code(proj), stream()))  # fmt: skip
    return out


def rotary_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """(cos, sin) of position * inv_freq[i] for every token, float32 [T, len(inv_freq), 2]: made once
    per step for all the layers that rotate by the same frequencies."""
    require_cuda(positions, inv_freq)
    if positions.dtype != torch.int32 or inv_freq.dtype != torch.float32 or not positions.is_contiguous() or not inv_freq.is_contiguous():
        raise KernelLibraryError("rotary_table takes contiguous int32 positions and float32 frequencies")
    table = torch.empty(positions.shape[0], inv_freq.shape[0], 2, device=positions.device, dtype=torch.float32)
    check(lib().asb_rotary_table(ptr(table), ptr(positions), ptr(inv_freq), positions.shape[0], inv_freq.shape[0], stream()))
    return table


def linear_recurrence(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, state: torch.Tensor,
                      state_slots: torch.Tensor, req_q_start: torch.Tensor, num_requests: int, *,
                      decay: torch.Tensor | None = None, token_decay: torch.Tensor | None = None,
                      token_gain: torch.Tensor | None = None, norm_state: torch.Tensor | None = None,
                      positions: torch.Tensor | None = None, inv_freq: torch.Tensor | None = None, rotary_dim: int = 0,
                      q_scale: float = 1.0, k_scale: float = 1.0, activation: bool = False,
                      segments: Segments | None = None, table: torch.Tensor | None = None,
                      qk_share: int = 1) -> tuple[torch.Tensor, torch.Tensor | None]:  # fmt: skip
    """The general form of `lightning_attention`: S_t = a_t S_(t-1) + b_t k_t v_t^T, o_t = S_t^T q_t.

    a: `decay` float32 [H], or `token_decay` float32 [T, H]; b: `token_gain` float32 [T, H], or 1.
    `norm_state` float32 [slots, H, D]: a normaliser n_t = a_t n_(t-1) + b_t k_t is kept there too and
    n_t . q_t returned as the second result, float32 [T, H]. `positions` int32 [T] with `inv_freq`
    float32 [rotary_dim / 2]: q and k are rotated first, pairs (i, i + rotary_dim / 2) of each head's
    first rotary_dim entries by position * inv_freq[i] (`table`: the step's `rotary_table` of these
    positions and frequencies, where the caller has made it already). q_scale and k_scale multiply q
    and k after that. `qk_share`: every group of this many neighbouring heads reads one q and one k
    (proj then holds H / qk_share heads of D columns from q_off and from k_off); values, states and
    outputs stay per head. Everything from the rotation on is float32. Returns (o float32 [T, H * V], n . q or None)."""
    require_cuda(proj, state, state_slots, req_q_start, decay, token_decay, token_gain, norm_state, positions, inv_freq)
    if proj.dim() != 2 or not proj.is_contiguous():
        raise KernelLibraryError("linear_recurrence: proj must be a contiguous [tokens, columns] tensor")
    if state.dtype != torch.float32 or state.dim() != 4 or not state.is_contiguous():
        raise KernelLibraryError("linear_recurrence: state must be contiguous float32 [slots, H, D, V]")
    T = proj.shape[0]
    _, H, D, V = state.shape
    if (decay is None) == (token_decay is None):
        raise KernelLibraryError("linear_recurrence: give one of decay [H] and token_decay [T, H]")
    for t, shape, name in ((decay, (H,), "decay"), (token_decay, (T, H), "token_decay"), (token_gain, (T, H), "token_gain"),
                           (norm_state, (state.shape[0], H, D), "norm_state"), (inv_freq, (rotary_dim // 2,), "inv_freq")):  # fmt: skip
        if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous()):
            raise KernelLibraryError(f"linear_recurrence: {name} must be contiguous float32 {list(shape)}")
    for t in (state_slots, req_q_start, positions):
        if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
            raise KernelLibraryError("linear_recurrence: index tensors must be contiguous int32")
    if positions is not None and (rotary_dim % 2 or rotary_dim > D or inv_freq is None or positions.shape[0] < T):
        raise KernelLibraryError(f"linear_recurrence: cannot rotate {rotary_dim} of {D} entries")
    if qk_share < 1 or H % qk_share or (qk_share > 1 and (norm_state is not None or positions is not None)):
        raise KernelLibraryError(f"linear_recurrence: {H} heads sharing q and k in groups of {qk_share} (no normaliser, no rotation then)")
    if max(q_off, k_off) + H // qk_share * D > proj.shape[1] or v_off + H * V > proj.shape[1]:
        raise KernelLibraryError("linear_recurrence: the column ranges lie outside proj")
    out = torch.empty(T, H * V, device=proj.device, dtype=torch.float32)
    nq = torch.empty(T, H, device=proj.device, dtype=torch.float32) if norm_state is not None else None
    rot = rotary_dim if positions is not None else 0
    if rot and table is None:
        table = rotary_table(positions[:T], inv_freq)
    if rot and (table.dtype != torch.float32 or tuple(table.shape) != (T, rot // 2, 2) or not table.is_contiguous()):
        raise KernelLibraryError(f"linear_recurrence: the rotation table must be contiguous float32 [{T}, {rot // 2}, 2]")

    through = None  # with per-token decays: what is left of a state after each segment

    def run(state_, slots_, starts_, norm_state_, count, mode):
        check(lib().asb_linear_recurrence_shared(ptr(out), ptr(proj), proj.shape[1], q_off, k_off, v_off, ptr(state_), ptr(slots_),
                                                 ptr(starts_), ptr(decay), ptr(token_decay), ptr(token_gain), ptr(norm_state_),
                                                 ptr(nq), ptr(through), ptr(table) if rot else None, rot, float(q_scale),
                                                 float(k_scale), count, H, D, V, int(activation), mode, qk_share,
                                                 dtype_code(proj), stream()))  # fmt: skip

    if segments is None:
        run(state, state_slots, req_q_start, norm_state, num_requests, 0)
        return out, nq
    local = torch.empty(segments.count, H, D, V, device=proj.device, dtype=torch.float32)
    local_n = torch.empty(segments.count, H, D, device=proj.device, dtype=torch.float32) if norm_state is not None else None
    if token_decay is not None:
        through = torch.empty(segments.count, H, device=proj.device, dtype=torch.float32)
    run(local, segments.index, segments.bounds, local_n, segments.count, 1)
    for own, kept, v in ((local, state, V), (local_n, norm_state, 1)):
        if own is not None:
            check(lib().asb_recurrence_scan(ptr(own), ptr(kept), ptr(state_slots), ptr(segments.req_start), ptr(segments.bounds),
                                            ptr(decay), ptr(through), num_requests, H, D, v, stream()))  # fmt: skip
    run(local, segments.index, segments.bounds, local_n, segments.count, 2)
    return out, nq
