"""Differential attention as a mixer: every head holds two score maps over the same values, each a
softmax attention of its own, and gives their difference.

q = Wq h has heads x 2 x dim rows and k = Wk h has kv_heads x 2 x dim, head by head as
[map 1, map 2]; v = Wv h has kv_heads x vdim. With a1, a2 the two maps' outputs per head and
lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (four learned vectors of `dim` entries, one number
per layer): o = a1 - lambda a2, divided by its root mean square over vdim (no gain) and
multiplied by 1 - diff; then the output projection. A position encoding turns the first entries
of every map of q and k. `chunk`: a query sees only the keys of its own run of that many
positions; `window`: only its last that many.

How it runs: the two maps of a head become two query heads of the head's group, each with its
`dim` entries at its own offset among zeros, and a key head holds its two maps side by side, so a
query head's product with the key head is its own map's score. The paged attention kernels then
serve 2 x heads query heads over kv_heads key and value heads, with one copy of the values, at a
head size of max(2 dim, vdim).
"""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, KVCacheSpec, Mixer, PageSpec, StepContext, build_part, register_part
from atomserve_b200.parts.spec import PartSpec, TensorSpec

MAPS = 2


class DifferentialAttention(Mixer):
    def __init__(self, hidden_size: int, prefix: str, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                 scale: float, diff: float, eps: float, position: PartSpec | None = None, chunk: int | None = None,
                 window: int | None = None):  # fmt: skip
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.prefix = hidden_size, prefix
        self.num_heads, self.num_kv_heads, self.dim, self.value_dim = num_heads, num_kv_heads, head_dim, value_dim
        self.head_dim = max(MAPS * head_dim, value_dim)  # what pages and kernels run at
        self.scale, self.diff, self.eps = float(scale), float(diff), float(eps)
        self.chunk, self.window = chunk, window
        self.position = build_part("position", position, hidden_size) if position else None
        self.qkv_proj = self.o_proj = None
        self.lam = 0.0

    def cache_spec(self) -> PageSpec:
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window, self.chunk)

    def tensor_specs(self) -> list[TensorSpec]:
        p, d = self.prefix, self.hidden_size
        specs = [
            TensorSpec(p + "q", (self.num_heads * MAPS * self.dim, d)),
            TensorSpec(p + "k", (self.num_kv_heads * MAPS * self.dim, d)),
            TensorSpec(p + "v", (self.num_kv_heads * self.value_dim, d)),
            TensorSpec(p + "o", (d, self.num_heads * self.value_dim)),
        ]
        return specs + [TensorSpec(p + n, (self.dim,), kind="gain", init="normal") for n in ("lq1", "lk1", "lq2", "lk2")]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p = self.prefix
        self.qkv_proj = torch.cat([tensors[p + "q"], tensors[p + "k"], tensors[p + "v"]]).contiguous()
        self.o_proj = tensors[p + "o"]
        lq1, lk1, lq2, lk2 = (tensors[p + n].float() for n in ("lq1", "lk1", "lq2", "lk2"))
        # one number per layer, float32, made once
        self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + self.diff)
        if self.position is not None:
            self.position.prepare(self.o_proj.device)
            rotary = self.position.fused_rotary()
            if rotary is None or rotary.pairing != "half" or rotary.magnitude != 1.0:
                raise NotImplementedError("differential attention turns pairs (i, i + rotary_dim / 2) by position x frequency")

    def attend(self, h: torch.Tensor, ctx: StepContext, cache: CacheView, write_cache: bool) -> torch.Tensor:
        """The heads' normed differences side by side, [T, heads * vdim]."""
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        rotary = self.position.fused_rotary() if self.position is not None else None
        proj = ops.linear(h, self.qkv_proj if write_cache else self.qkv_proj[: H * MAPS * self.dim])
        q = ops.qk_prepare_store(
            proj, H, KV, MAPS, self.dim, self.value_dim, hd, ctx.positions,
            inv_freq=rotary.inv_freq if rotary else None, rotary_dim=rotary.rotary_dim if rotary else 0,
            slots=cache.slots if write_cache else None, k_cache=cache.k if write_cache else None,
            v_cache=cache.v if write_cache else None,
        )  # fmt: skip
        maps = ops.paged_attention(
            q, cache.k, cache.v, cache.block_tables, ctx.req_q_start, ctx.req_pos_start,
            num_requests=ctx.num_requests, max_context=ctx.max_context, window=self.window, scale=self.scale,
            host_q_lens=ctx.host_q_lens or None, chunk=self.chunk,
        )  # fmt: skip
        return ops.differential_combine(maps, self.value_dim, self.lam, 1.0 - self.diff, self.eps)

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext,
                cache: CacheView | None, write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        mixed = self.attend(h, ctx, cache, write_cache)
        return ops.linear(mixed, self.o_proj, residual, out_dtype=torch.float32 if residual is None else None)


register_part("mixer", "differential_attention", DifferentialAttention)
