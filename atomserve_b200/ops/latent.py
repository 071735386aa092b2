"""Attention over a cached low-rank latent (csrc/latent_attention.cu): the per-token cache
write with the queries' rotation, the per-head products, and the attention."""

from __future__ import annotations

import ctypes
import os

import torch

from atomserve_b200.ops.attention import TARGET_BLOCKS
from atomserve_b200.ops.library import FLOAT32, KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream


# Which kernel serves bfloat16 pages: "mma" (tensor cores, csrc/latent_attention_mma.cu; the default
# where its sizes hold) or "simt" (the CUDA-core kernel that float32 always runs).
ATTENTION_KERNEL = os.environ.get("ATOMSERVE_B200_LATENT_ATTENTION", "mma")


def latent_prepare(proj: torch.Tensor, q_off: int, kv_off: int | None, q_lat: torch.Tensor, pages: torch.Tensor | None,
                   gain: torch.Tensor | None, inv_freq: torch.Tensor | None, positions: torch.Tensor,
                   slots: torch.Tensor | None, *, heads: int, dim: int, rank: int, rot: int, rot_dims: int,
                   eps: float) -> None:  # fmt: skip
    """Per token of proj [T, W]: with `pages` ([num_blocks, 1, block_size, rank + rot]), write
    [rms_norm(latent) * gain | turned shared key part] to the token's slot, the latent being the
    `rank` columns from kv_off and the key part the `rot` after them; and turn the last `rot` of
    each head's dim + rot query columns (from q_off) into q_lat[t, h, rank:] (float32). Of the
    `rot` entries the first `rot_dims` turn, neighbours paired (rot 0: no such part, no frequencies)."""
    require_cuda(proj, q_lat, pages, gain, inv_freq, positions, slots)
    if proj.dim() != 2 or not proj.is_contiguous():
        raise KernelLibraryError("latent_prepare: proj must be a contiguous [tokens, columns] tensor")
    T = proj.shape[0]
    if q_lat.dtype != torch.float32 or q_lat.shape != (T, heads, rank + rot) or not q_lat.is_contiguous():
        raise KernelLibraryError(f"latent_prepare: q_lat must be contiguous float32 [{T}, {heads}, {rank + rot}]")
    if rot_dims and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.shape != (rot_dims // 2,)):
        raise KernelLibraryError(f"latent_prepare: inv_freq must be float32 [{rot_dims // 2}]")
    if pages is not None:
        if pages.dtype != proj.dtype or pages.dim() != 4 or pages.shape[1] != 1 or pages.shape[3] != rank + rot or not pages.is_contiguous():
            raise KernelLibraryError("latent_prepare: pages must be [num_blocks, 1, block_size, rank + rot] in proj's dtype")
        if gain is None or gain.dtype != torch.float32 or gain.shape != (rank,) or slots is None or kv_off is None:
            raise KernelLibraryError("latent_prepare: storing needs the latent's gain, its columns and the slots")
    check(lib().asb_latent_prepare(ptr(proj), proj.shape[1], q_off, kv_off or 0, ptr(q_lat), ptr(pages), ptr(gain),
                                   ptr(inv_freq), ptr(positions), ptr(slots), T, heads, dim, rank, rot, rot_dims,
                                   float(eps), dtype_code(proj), stream()))  # fmt: skip


def head_matmul_on_tensor_cores(w: torch.Tensor, k: int) -> bool:
    """Whether per-head products with this weight dtype and inner size run the tensor-core kernel,
    which takes the weights as [H, N, K]."""
    return ATTENTION_KERNEL == "mma" and w.dtype == torch.bfloat16 and k % 8 == 0


def head_matmul(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: torch.Tensor | None = None,
                w_is_nk: bool = False) -> torch.Tensor:  # fmt: skip
    """out[t, h, :] = x[t, h, :] . w[h], times sigmoid(gate[t, h]) where a gate is given. w is
    [H, K, N] in the compute dtype, or with `w_is_nk` [H, N, K] in bfloat16 (the tensor-core
    kernel's layout). x [T, H, K] and out [T, H, N] are float32 or the compute dtype and may be
    strided views with unit stride along the last axis."""
    require_cuda(x, w, out, gate)
    H, K, N = (w.shape[0], w.shape[2], w.shape[1]) if w_is_nk else w.shape
    T = x.shape[0]
    if x.shape != (T, H, K) or out.shape != (T, H, N) or x.stride(2) != 1 or out.stride(2) != 1 or not w.is_contiguous():
        raise KernelLibraryError(f"head_matmul: x {tuple(x.shape)} . w {tuple(w.shape)} -> out {tuple(out.shape)}")
    for t in (x, out):
        if t.dtype not in (torch.float32, w.dtype):
            raise KernelLibraryError("head_matmul: x and out are float32 or w's dtype")
    if gate is not None and (gate.shape != (T, H) or gate.dtype != w.dtype or gate.stride(1) != 1):
        raise KernelLibraryError("head_matmul: gate must be [T, H] in w's dtype with unit column stride")
    if w_is_nk:
        if not head_matmul_on_tensor_cores(w, K) or w.data_ptr() % 16:
            raise KernelLibraryError("head_matmul: [H, N, K] weights are bfloat16 with K a multiple of 8")
        check(lib().asb_head_matmul_mma(ptr(out), int(out.dtype == torch.float32), out.stride(0), out.stride(1), ptr(x),
                                        int(x.dtype == torch.float32), x.stride(0), x.stride(1), ptr(w), ptr(gate),
                                        gate.stride(0) if gate is not None else 0, T, H, K, N, stream()))  # fmt: skip
        return out
    check(lib().asb_head_matmul(ptr(out), int(out.dtype == torch.float32), out.stride(0), out.stride(1), ptr(x),
                                int(x.dtype == torch.float32), x.stride(0), x.stride(1), ptr(w), ptr(gate),
                                gate.stride(0) if gate is not None else 0, T, H, K, N, dtype_code(w), stream()))  # fmt: skip
    return out


def latent_tile_shape(heads: int) -> tuple[int, int]:
    qt, gc = ctypes.c_int(), ctypes.c_int()
    lib().asb_latent_attention_tile_shape(heads, ctypes.byref(qt), ctypes.byref(gc))
    return qt.value, gc.value


def plan_latent_partitions(num_tokens: int, num_requests: int, heads: int, max_context: int) -> tuple[int, int]:
    """(partition size, partitions): the keys are split only when the step's query tiles alone
    cannot fill the device. Partitions are aligned to absolute key positions."""
    qt, gc = latent_tile_shape(heads)
    blocks = (-(-num_tokens // qt) + num_requests) * -(-heads // gc)
    if blocks >= TARGET_BLOCKS or max_context <= 256:
        return 1 << 30, 1
    want = -(-TARGET_BLOCKS // blocks)
    size = max(256, -(-(-(-max_context // want)) // 256) * 256)
    parts = (max_context - 1) // size + 1
    return (size, parts) if parts > 1 else (1 << 30, 1)


def latent_attention(q_lat: torch.Tensor, pages: torch.Tensor, block_tables: torch.Tensor, req_q_start: torch.Tensor,
                     req_pos_start: torch.Tensor, *, rank: int, num_requests: int, max_context: int, scale: float,
                     partitions: tuple[int, int] | None = None, window: int | None = None) -> torch.Tensor:  # fmt: skip
    """Causal softmax attention of q_lat [T, H, rank + rot] (float32) over the requests' cached
    [c | kr] vectors; returns sum_j p_j c_j as float32 [T, H, rank]. With a `window` a query at
    position p sees the keys j with 0 <= p - j < window."""
    require_cuda(q_lat, pages, block_tables, req_q_start, req_pos_start)
    T, H, Dk = q_lat.shape
    if q_lat.dtype != torch.float32 or not q_lat.is_contiguous() or pages.shape[3] != Dk or pages.shape[1] != 1:
        raise KernelLibraryError("latent_attention: q_lat float32 [T, H, Dk] against pages [blocks, 1, bs, Dk]")
    for t in (block_tables, req_q_start, req_pos_start):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelLibraryError("latent_attention: index tensors must be contiguous int32")
    out = torch.empty(T, H, rank, device=q_lat.device, dtype=torch.float32)
    win = int(window) if window else 0
    ps, np_ = partitions or plan_latent_partitions(T, num_requests, H, max_context)
    part_m = part_l = part_acc = None
    if np_ > 1:
        part_m = torch.empty(T * H * np_, device=out.device, dtype=torch.float32)
        part_l = torch.empty_like(part_m)
        part_acc = torch.empty(T * H * np_ * rank, device=out.device, dtype=torch.float32)
    if ATTENTION_KERNEL == "mma" and pages.dtype == torch.bfloat16 and lib().asb_latent_attention_mma_supported(rank, Dk - rank):
        check(lib().asb_latent_attention_mma(ptr(out), ptr(q_lat), ptr(pages), ptr(block_tables), ptr(req_q_start),
                                             ptr(req_pos_start), ptr(part_m), ptr(part_l), ptr(part_acc), T, num_requests, H,
                                             rank, Dk - rank, pages.shape[2], block_tables.shape[1], ps, np_, float(scale),
                                             win, stream()))  # fmt: skip
    else:
        check(lib().asb_latent_attention(ptr(out), ptr(q_lat), ptr(pages), ptr(block_tables), ptr(req_q_start),
                                         ptr(req_pos_start), ptr(part_m), ptr(part_l), ptr(part_acc), T, num_requests, H, rank,
                                         Dk - rank, pages.shape[2], block_tables.shape[1], ps, np_, float(scale),
                                         win, dtype_code(pages), stream()))  # fmt: skip
    if np_ > 1:
        check(lib().asb_attention_reduce(ptr(out), ptr(part_m), ptr(part_l), ptr(part_acc), T * H, np_, rank, FLOAT32, stream()))
    return out
