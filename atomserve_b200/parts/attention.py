"""Grouped-query attention over cache pages, with optional per-head RMSNorm of q and k before
the position encoding (Qwen3's form, atomserve/model.py:292-336), an optional sliding window,
and no biases. Sizes, eps, the position encoding, the score scale and the window are parameters;
`names` gives the checkpoint's tensor names where they are not the `*_proj.weight` ones, and
`value_dim` a value size that differs from the key size.

Where value_dim != head_dim the pages and kernels run at the larger of the two: the narrower of
(queries and keys) and (values) is padded with zero rows in the loaded weights, which changes no
score and no output (the q/k norm's mean is taken over head_dim entries: the gains carry
sqrt(head_dim / padded) and the kernel's eps is eps * head_dim / padded, the same quotient)."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, KVCacheSpec, Mixer, Norm, PageSpec, StepContext, build_part, register_part
from atomserve_b200.parts.spec import PartSpec, TensorSpec


class GQAttention(Mixer):
    def __init__(
        self,
        hidden_size: int,
        prefix: str,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        qk_norm_eps: float | None = None,
        position: PartSpec | None = None,
        window: int | None = None,
        scale: float | None = None,
        value_dim: int | None = None,
        names: dict[str, str] | None = None,
        sink: bool = False,
        softcap: float | None = None,
        query_temperature: tuple[float, int] | None = None,
        chunk: int | None = None,
    ):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.prefix = hidden_size, prefix
        # key_dim and value_dim: the checkpoint's sizes; head_dim: what pages and kernels run at
        self.key_dim, self.value_dim = head_dim, (head_dim if value_dim is None else value_dim)
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, max(self.key_dim, self.value_dim)
        n = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight", q_norm="q_norm.weight", k_norm="k_norm.weight",
                 sink="sink")
        n.update(names or {})
        self.names = {key: prefix + value for key, value in n.items()}
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else head_dim**-0.5
        self.position = build_part("position", position, hidden_size) if position else None
        # `sink`: a learned logit per head in the softmax's denominator; `softcap`: scores become
        # softcap tanh(score / softcap); `query_temperature=(coef, every)`: queries at position p are
        # multiplied by 1 + coef ln(floor((p + 1) / every) + 1); `chunk`: a query sees only the keys of
        # its own run of that many positions
        self.has_sink, self.softcap, self.chunk = bool(sink), (float(softcap) if softcap else None), chunk
        self.query_temperature = (float(query_temperature[0]), int(query_temperature[1])) if query_temperature else None
        if self.query_temperature is not None and (qk_norm_eps is not None or self.query_temperature[1] < 1):
            raise ValueError("a query temperature goes with unnormed queries and a positive period")
        self.qkv_proj = self.o_proj = self.q_gain = self.k_gain = self.sink = None

    def cache_spec(self) -> PageSpec:
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window, self.chunk)

    def tensor_specs(self) -> list[TensorSpec]:
        n, d, kd, vd = self.names, self.hidden_size, self.key_dim, self.value_dim
        specs = [
            TensorSpec(n["q"], (self.num_heads * kd, d)),
            TensorSpec(n["k"], (self.num_kv_heads * kd, d)),
            TensorSpec(n["v"], (self.num_kv_heads * vd, d)),
            TensorSpec(n["o"], (d, self.num_heads * vd)),
        ]
        if self.qk_norm_eps is not None:
            specs += [
                TensorSpec(n["q_norm"], (kd,), kind="gain", init="gain"),
                TensorSpec(n["k_norm"], (kd,), kind="gain", init="gain"),
            ]
        if self.has_sink:
            specs.append(TensorSpec(n["sink"], (self.num_heads,), kind="gain", init="normal"))
        return specs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        n, hd, kd, vd = self.names, self.head_dim, self.key_dim, self.value_dim

        def rows_per_head(w: torch.Tensor, heads: int, size: int) -> torch.Tensor:
            if size == hd:
                return w
            padded = w.new_zeros(heads, hd, w.shape[1])
            padded[:, :size] = w.view(heads, size, w.shape[1])
            return padded.view(heads * hd, w.shape[1])

        # q, k and v stacked along the output rows: one product instead of three
        # (atomserve/loader.py:112-116)
        self.qkv_proj = torch.cat([rows_per_head(tensors[n["q"]], self.num_heads, kd),
                                   rows_per_head(tensors[n["k"]], self.num_kv_heads, kd),
                                   rows_per_head(tensors[n["v"]], self.num_kv_heads, vd)]).contiguous()  # fmt: skip
        self.o_proj = tensors[n["o"]]
        if vd != hd:  # the padded value entries are zero: their columns of the output projection too
            o = self.o_proj.new_zeros(self.o_proj.shape[0], self.num_heads, hd)
            o[:, :, :vd] = self.o_proj.view(-1, self.num_heads, vd)
            self.o_proj = o.view(-1, self.num_heads * hd).contiguous()
        self.sink = tensors[n["sink"]].contiguous() if self.has_sink else None
        self.kernel_eps = self.qk_norm_eps
        if self.qk_norm_eps is not None:
            self.q_gain, self.k_gain = tensors[n["q_norm"]], tensors[n["k_norm"]]
            if kd != hd:
                pad = (kd / hd) ** 0.5
                self.q_gain = torch.cat([self.q_gain * pad, self.q_gain.new_zeros(hd - kd)]).contiguous()
                self.k_gain = torch.cat([self.k_gain * pad, self.k_gain.new_zeros(hd - kd)]).contiguous()
                self.kernel_eps = self.qk_norm_eps * kd / hd
        if self.position is not None:
            self.position.prepare(self.o_proj.device)
            rotary = self.position.fused_rotary()
            if rotary is not None and rotary.magnitude != 1.0:
                # cosines and sines times a constant: the turned entries of q and k times it, which
                # the gains of the norm before the rotation carry (a pair's two entries both turn)
                if self.qk_norm_eps is None:
                    raise NotImplementedError("a rotation with a magnitude needs the q/k norm, whose gains carry it")
                scale = torch.ones_like(self.q_gain)
                scale[: rotary.rotary_dim] = rotary.magnitude
                self.q_gain, self.k_gain = (self.q_gain * scale).contiguous(), (self.k_gain * scale).contiguous()

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext,
                cache: CacheView | None, write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        # (no residual: a block that sums in float32 itself, and the product stays float32)
        return ops.linear(self.attend(h, ctx, cache, write_cache), self.o_proj, residual,
                          out_dtype=torch.float32 if residual is None else None)  # fmt: skip

    def forward_then(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache: CacheView | None,
                     write_cache: bool, then: Norm) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
        after_linear = getattr(then, "after_linear", None)
        if after_linear is None:
            return super().forward_then(h, residual, ctx, cache, write_cache, then)
        return after_linear(self.attend(h, ctx, cache, write_cache), self.o_proj, residual)

    def forward_for_stream(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool = True):
        """mix(h) for a block that adds it to a float32 stream itself: float32, or the output
        projection's partial sums for the norm that follows to add up (`ops.linear_for_stream`)."""
        return ops.linear_for_stream(self.attend(h, ctx, cache, write_cache), self.o_proj)

    def attend(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool) -> torch.Tensor:
        """The heads' outputs side by side, [T, H * hd], before the output projection."""
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        # the position encoding says how it is applied: by the fused kernel below (a rotation by
        # position x frequency), or by its own `encode` on the normalised queries and keys
        rotary = self.position.fused_rotary() if self.position is not None else None
        if rotary is not None and rotary.pairing != "half":
            raise NotImplementedError("this attention's fused kernel turns pairs (i, i + rotary_dim / 2) only")
        if self.position is not None and rotary is None:
            q = self._project_encode_store(h, ctx, cache, write_cache)
        elif self.query_temperature is not None:
            # unnormed queries scaled by position: the kernel for heads of several maps, with one map
            # (the padded rows of the stacked weight give the zeros of the wider head size)
            qkv = ops.linear(h, self.qkv_proj if write_cache else self.qkv_proj[: H * hd])
            q = ops.qk_prepare_store(
                qkv, H, KV, 1, hd, hd, hd, ctx.positions,
                inv_freq=rotary.inv_freq if rotary else None, rotary_dim=rotary.rotary_dim if rotary else 0,
                temperature=self.query_temperature, slots=cache.slots if write_cache else None,
                k_cache=cache.k if write_cache else None, v_cache=cache.v if write_cache else None,
            )  # fmt: skip
        else:
            # reading another entry's keys and values, only queries are projected
            weight, kv_heads = (self.qkv_proj, KV) if write_cache else (self.qkv_proj[: H * hd], 0)
            qkv = None
            if ops.qk_norm_rope_store_takes_partial(hd, rotary.rotary_dim if rotary else None):
                # with few tokens the product stays as the GEMM's partial sums and the next kernel adds them up
                qkv = ops.linear_partial(h, weight)
            if qkv is None:
                qkv = ops.linear(h, weight)
            q = ops.qk_norm_rope_store(
                qkv, H, kv_heads, hd, ctx.positions,
                q_gain=self.q_gain, k_gain=self.k_gain, eps=self.kernel_eps or 0.0,
                inv_freq=rotary.inv_freq if rotary else None, rotary_dim=rotary.rotary_dim if rotary else 0,
                slots=cache.slots if write_cache else None,
                k_cache=cache.k if write_cache else None, v_cache=cache.v if write_cache else None,
            )  # fmt: skip
        out = ops.paged_attention(
            q, cache.k, cache.v, cache.block_tables, ctx.req_q_start, ctx.req_pos_start,
            num_requests=ctx.num_requests, max_context=ctx.max_context, window=self.window,
            scale=self.scale, host_q_lens=ctx.host_q_lens or None, sink=self.sink, chunk=self.chunk, softcap=self.softcap,
        )  # fmt: skip
        return out.view(-1, H * hd)


    def _project_encode_store(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool) -> torch.Tensor:
        """The path for an encoding that is no fused rotation: the same kernel normalises q and k
        without turning or storing them, the encoding's `encode` works the positions in, and a
        second pass of the kernel (no norm, no rotation) writes keys and values to their pages."""
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        T = h.shape[0]
        kv_heads = KV if write_cache else 0
        qkv = ops.linear(h, self.qkv_proj if write_cache else self.qkv_proj[: H * hd])
        normed = qkv
        if self.qk_norm_eps is not None:
            heads = qkv.view(T, H + 2 * kv_heads, hd)
            q = ops.rms_norm(heads[:, :H].reshape(T * H, hd), self.q_gain, self.kernel_eps).view(T, H, hd)
            k = ops.rms_norm(heads[:, H : H + kv_heads].reshape(T * kv_heads, hd), self.k_gain, self.kernel_eps).view(T, kv_heads, hd) if kv_heads else None
        else:
            heads = qkv.view(T, H + 2 * kv_heads, hd)
            q, k = heads[:, :H].contiguous(), (heads[:, H : H + kv_heads].contiguous() if kv_heads else None)
        q, k = self.position.encode(q, k, ctx)
        if not write_cache:
            return q.contiguous()
        normed = torch.cat([q.reshape(T, H * hd), k.reshape(T, KV * hd), qkv[:, (H + KV) * hd :]], dim=1)
        return ops.qk_norm_rope_store(normed, H, KV, hd, ctx.positions, q_gain=None, k_gain=None, eps=0.0, inv_freq=None,
                                      rotary_dim=0, slots=cache.slots, k_cache=cache.k, v_cache=cache.v)  # fmt: skip


register_part("mixer", "gqa_attention", GQAttention)
