"""Softmax attention over a cached low-rank latent, as a mixer.

Per token a down-projection gives `kv_rank` values, RMS-normed into the latent c, and `rot_dim`
values that, position-encoded, are a key part kr shared by all heads; [c | kr] is all that is
cached. Head h's keys and values are up-projections of c (Wuk_h c with kr behind it, Wuv_h c),
its queries `dim` plain and `rot_dim` position-encoded values. The up-projections are applied
on the query side (scores against c itself, the weighted sum of c up-projected afterwards), so
the pages are read as they are. A sigmoid gate per head, projected from the same input,
multiplies the head's output before the output projection.

`rot_dim=0` with no position encoding is the form without a position-encoded part; `gated=False`
the form without the gate; with `window` a query sees its last `window` positions only (itself
included) and pages the window has passed are given back.

A mixer built with `reads_cache_of_another=True` has no down-projection: the run order gives
it the pages of an earlier latent-attention entry (`LayerCall.cache_from`), which it reads with
its own queries and up-projections.
"""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, Mixer, PageSpec, PageTensor, StepContext, build_part, register_part
from atomserve_b200.parts.spec import PartSpec, TensorSpec

PAGE = "latent"


class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, prefix: str, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 scale: float, eps: float, position: PartSpec | None = None, reads_cache_of_another: bool = False,
                 gated: bool = True, window: int | None = None):  # fmt: skip
        if (rot_dim > 0) != (position is not None):
            raise ValueError("a position-encoded key part needs a position encoding, and the other way round")
        self.hidden_size, self.prefix = hidden_size, prefix
        self.heads, self.dim, self.rot_dim, self.vdim, self.kv_rank = heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.eps, self.reads_only = float(scale), float(eps), reads_cache_of_another
        self.gated, self.window = gated, window
        self.position = build_part("position", position, hidden_size) if position is not None else None
        self.in_proj = self.uk = self.uv_t = self.o_proj = self.latent_gain = None

    def cache_spec(self) -> PageSpec | None:
        if self.reads_only:
            return None
        return PageSpec((PageTensor(PAGE, 1, self.kv_rank + self.rot_dim),), self.window)

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, H = self.prefix, self.hidden_size, self.heads
        specs = [
            TensorSpec(p + "q", (H * (self.dim + self.rot_dim), d)),
            TensorSpec(p + "uk", (H * self.dim, self.kv_rank)),
            TensorSpec(p + "uv", (H * self.vdim, self.kv_rank)),
            TensorSpec(p + "o", (d, H * self.vdim)),
        ] + ([TensorSpec(p + "g", (H, d))] if self.gated else [])
        if not self.reads_only:
            specs += [
                TensorSpec(p + "dkv", (self.kv_rank + self.rot_dim, d)),
                TensorSpec(p + "dkv.norm", (self.kv_rank,), kind="gain", init="gain"),
            ]
        return specs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p, H = self.prefix, self.heads
        # queries, (down-projection,) gates stacked along the output rows: one product
        rows = [tensors[p + "q"]] + ([] if self.reads_only else [tensors[p + "dkv"]]) + ([tensors[p + "g"]] if self.gated else [])
        self.in_proj = torch.cat(rows).contiguous()
        # per head, keys' up-projection [dim, rank] (absorbed into the queries) and values' [rank, vdim];
        # the tensor-core kernel takes each with its inner size last instead
        uk, uv = tensors[p + "uk"].view(H, self.dim, self.kv_rank), tensors[p + "uv"].view(H, self.vdim, self.kv_rank)
        self.uk_nk = ops.head_matmul_on_tensor_cores(uk, self.dim)
        self.uv_nk = ops.head_matmul_on_tensor_cores(uv, self.kv_rank)
        self.uk = (uk.transpose(1, 2) if self.uk_nk else uk).contiguous()
        self.uv_t = (uv if self.uv_nk else uv.transpose(1, 2)).contiguous()
        self.o_proj = tensors[p + "o"]
        self.latent_gain = None if self.reads_only else tensors[p + "dkv.norm"]
        self.rotary = None
        if self.position is not None:
            self.position.prepare(self.o_proj.device)
            rotary = self.position.fused_rotary()
            if rotary is None or rotary.pairing != "interleaved" or rotary.rotary_dim > self.rot_dim or rotary.magnitude != 1.0:
                raise ValueError("latent attention turns neighbouring pairs of its position-encoded part by position x frequency")
            self.rotary = rotary

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext,
                cache: CacheView | None, write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        # without a residual (a block that sums in float32 itself) the product stays float32
        return ops.linear(self.mixed(h, ctx, cache, write_cache), self.o_proj, residual,
                          out_dtype=torch.float32 if residual is None else None)  # fmt: skip

    def forward_for_stream(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool = True):
        """mix(h) for a block that adds it to a float32 stream and norms the sum at once: float32, or
        the output projection's partial sums for that norm to add up (`ops.linear_for_stream`)."""
        return ops.linear_for_stream(self.mixed(h, ctx, cache, write_cache), self.o_proj)

    def mixed(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool) -> torch.Tensor:
        """The gated heads' outputs side by side, [T, heads * vdim], before the output projection."""
        if write_cache == self.reads_only:
            raise ValueError("a latent attention without a down-projection reads another entry's pages, one with it its own")
        T, H, D, Rt, V, R = h.shape[0], self.heads, self.dim, self.rot_dim, self.vdim, self.kv_rank
        q_cols = H * (D + Rt)
        gate_off = q_cols + (0 if self.reads_only else R + Rt)
        proj = ops.linear(h, self.in_proj)
        pages = cache.pages[PAGE]
        q_lat = torch.empty(T, H, R + Rt, device=h.device, dtype=torch.float32)
        ops.head_matmul(proj[:, :q_cols].view(T, H, D + Rt)[:, :, :D], self.uk, q_lat[:, :, :R], w_is_nk=self.uk_nk)
        ops.latent_prepare(proj, 0, None if self.reads_only else q_cols, q_lat, None if self.reads_only else pages,
                           self.latent_gain, self.rotary.inv_freq if self.rotary else None, ctx.positions,
                           None if self.reads_only else cache.slots, heads=H, dim=D, rank=R, rot=Rt,
                           rot_dims=self.rotary.rotary_dim if self.rotary else 0, eps=self.eps)  # fmt: skip
        mixed = ops.latent_attention(q_lat, pages, cache.block_tables, ctx.req_q_start, ctx.req_pos_start, rank=R,
                                     num_requests=ctx.num_requests, max_context=ctx.max_context, scale=self.scale,
                                     window=self.window)  # fmt: skip
        out = torch.empty(T, H * V, device=h.device, dtype=h.dtype)
        ops.head_matmul(mixed, self.uv_t, out.view(T, H, V), gate=proj[:, gate_off : gate_off + H] if self.gated else None,
                        w_is_nk=self.uv_nk)  # fmt: skip
        return out


register_part("mixer", "latent_attention", LatentAttention)
