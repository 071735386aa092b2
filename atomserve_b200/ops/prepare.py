"""Queries, keys and values of heads that hold several score maps on their way to the paged
attention kernels, and the maps' outputs joined afterwards: the Python faces of csrc/qk_prepare.cu."""

from __future__ import annotations

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream


def qk_prepare_store(proj: torch.Tensor, heads: int, kv_heads: int, maps: int, dim: int, vdim: int, head_dim: int,
                     positions: torch.Tensor, *, inv_freq: torch.Tensor | None = None, rotary_dim: int = 0,
                     temperature: tuple[float, int] | None = None, slots: torch.Tensor | None = None,
                     k_cache: torch.Tensor | None = None, v_cache: torch.Tensor | None = None) -> torch.Tensor:  # fmt: skip
    """proj [T, >= (heads + kv_heads) * maps * dim + kv_heads * vdim]: per row the queries
    [heads][maps][dim], keys [kv_heads][maps][dim] and values [kv_heads][vdim]. Every map of q and
    k has its first `rotary_dim` entries turned (pairs (i, i + rotary_dim / 2), angle position *
    inv_freq[i]); q is multiplied by 1 + coef ln(floor((position + 1) / every) + 1) for
    `temperature=(coef, every)`. Returns queries [T, heads * maps, head_dim] in which map j of head
    h is head h * maps + j with its entries at offset j * dim among zeros; keys go to their page
    as [kv_heads, head_dim] (a head's maps side by side, zeros behind) and values likewise, where
    `slots`, `k_cache` and `v_cache` are given (without them only queries are read)."""
    require_cuda(proj, positions, inv_freq, slots, k_cache, v_cache)
    if proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelLibraryError("qk_prepare_store: proj must be [tokens, columns] with unit column stride")
    T = proj.shape[0]
    if positions.dtype != torch.int32 or positions.shape[0] < T:
        raise KernelLibraryError("qk_prepare_store: positions must be int32, one per token")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.shape[0] * 2 < rotary_dim):
        raise KernelLibraryError("qk_prepare_store: inv_freq must be float32 [rotary_dim / 2]")
    bs = 0
    if k_cache is not None:
        if slots is None or v_cache is None or k_cache.shape != v_cache.shape or k_cache.dtype != proj.dtype or v_cache.dtype != proj.dtype:
            raise KernelLibraryError("qk_prepare_store: pages of keys and values of the projection's dtype, with slots")
        if k_cache.shape[1] != kv_heads or k_cache.shape[3] != head_dim or not k_cache.is_contiguous() or not v_cache.is_contiguous():
            raise KernelLibraryError(f"qk_prepare_store: pages must be [blocks, {kv_heads}, page, {head_dim}]")
        bs = k_cache.shape[2]
    q = torch.empty(T, heads * maps, head_dim, device=proj.device, dtype=proj.dtype)
    coef, every = temperature if temperature is not None else (0.0, 0)
    check(lib().asb_qk_prepare_store(ptr(proj), ptr(q), ptr(k_cache), ptr(v_cache), ptr(positions), ptr(slots),
                                     ptr(inv_freq), T, proj.stride(0), heads, kv_heads, maps, dim, vdim, head_dim,
                                     rotary_dim, bs, float(coef), int(every), dtype_code(proj), stream()))  # fmt: skip
    return q


def differential_combine(a: torch.Tensor, vdim: int, lam: float, post: float, eps: float) -> torch.Tensor:
    """a [T, 2 H, hd], the outputs of map 1 and map 2 of head h at 2h and 2h + 1: returns
    [T, H * vdim] with o = a1 - lam * a2 over the first vdim entries, o / sqrt(mean(o^2) + eps) * post."""
    require_cuda(a)
    T, heads2, hd = a.shape
    if heads2 % 2 or not a.is_contiguous():
        raise KernelLibraryError("differential_combine: a must be contiguous [tokens, 2 heads, head_dim]")
    out = torch.empty(T, heads2 // 2 * vdim, device=a.device, dtype=a.dtype)
    check(lib().asb_differential_combine(ptr(out), ptr(a), T * (heads2 // 2), hd, vdim, float(lam), float(post), float(eps),
                                         dtype_code(a), stream()))  # fmt: skip
    return out
