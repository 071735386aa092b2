"""The pre-norm residual arrangement: x = x + mixer(norm(x)); x = x + ff(norm(x))
(atomserve/model.py:11-13, 378-382). The residual additions happen inside the mixer's and the
feed-forward's last projection, so the block only routes tensors."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import Block, CacheView, Norm, StepContext, register_part


class PreNormBlock(Block):
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView | None,
                write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        return self.forward_chain(x, None, ctx, cache, write_cache, None)[0]

    def forward_chain(self, x: torch.Tensor, normed: torch.Tensor | None, ctx: StepContext, cache: CacheView | None,
                      write_cache: bool, then: Norm | None) -> tuple[torch.Tensor, torch.Tensor | None]:  # fmt: skip
        # each projection that ends a part is handed the norm that follows it, so that the part
        # may fuse the two (the norm after the feed-forward belongs to the next block)
        if normed is None:
            normed = self.mixer_norm.forward(x)
        x, normed = self.mixer.forward_then(normed, x, ctx, cache, write_cache, self.feed_forward_norm)
        if then is None:
            return self.feed_forward.forward(normed, x, ctx), None
        return self.feed_forward.forward_then(normed, x, ctx, then)


class PostNormBlock(Block):
    """The arrangement with the norm after the sum, over a float32 residual stream:
    x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ff(x)), the sublayers reading x itself
    (in the compute dtype). The norms are `StreamRMSNorm`s and carry alpha. A layer without a
    feed-forward (kind "none") ends after its first half. In a run of blocks the compute-dtype copy
    of x travels in the place where pre-norm blocks hand on the next block's normed input."""

    dtype = torch.float32  # the compute dtype, told by `bind_dtype` once the weights are loaded

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        super().load(tensors)
        self.has_feed_forward = not getattr(self.feed_forward, "absent", False)

    def bind_dtype(self, dtype: torch.dtype) -> None:
        self.dtype = dtype
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if hasattr(norm, "bind_dtype"):
                norm.bind_dtype(dtype)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView | None,
                write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        return self.forward_chain(x, None, ctx, cache, write_cache, None)[0]

    def forward_chain(self, x: torch.Tensor, normed: torch.Tensor | None, ctx: StepContext, cache: CacheView | None,
                      write_cache: bool, then: Norm | None) -> tuple[torch.Tensor, torch.Tensor | None]:  # fmt: skip
        h = normed if normed is not None else ops.cast_rows(x, self.dtype)
        # a sublayer that offers `forward_for_stream` may hand its last product over as the GEMM's
        # partial sums, which the norm's kernel then adds up itself (nothing runs in between)
        mix = getattr(self.mixer, "forward_for_stream", None)
        y = mix(h, ctx, cache, write_cache) if mix is not None else self.mixer.forward(h, None, ctx, cache, write_cache)
        x, h = self.mixer_norm.add_forward(x, y)
        if self.has_feed_forward:
            ff = getattr(self.feed_forward, "forward_for_stream", None)
            x, h = self.feed_forward_norm.add_forward(x, ff(h, ctx) if ff is not None else self.feed_forward.forward(h, None, ctx))
        return x, h


class OutputNormBlock(PostNormBlock):
    """The arrangement with the norm on each sublayer's output, over a float32 residual stream:
    x <- x + mult * norm1(mixer(x)); x <- x + mult * norm2(ff(x)), the sublayers reading x itself
    (in the compute dtype); the norms are `OutputNorm`s and carry mult and the layer scales. A
    layer without a feed-forward ends after its first half. A `token_input`, where the layer has
    one (`attach`), adds what it makes of the step's token ids after that. A mixer that offers
    `forward_halves` returns two outputs that the norm's kernel joins (two mixers side by side)."""

    token_input = None

    def attach(self, token_input) -> None:
        self.token_input = token_input

    def parts(self):
        return super().parts() + ([self.token_input] if self.token_input is not None else [])

    def bind_dtype(self, dtype: torch.dtype) -> None:
        super().bind_dtype(dtype)
        if self.token_input is not None:
            self.token_input.bind_dtype(dtype)

    def forward_chain(self, x: torch.Tensor, normed: torch.Tensor | None, ctx: StepContext, cache: CacheView | None,
                      write_cache: bool, then: Norm | None) -> tuple[torch.Tensor, torch.Tensor | None]:  # fmt: skip
        h = normed if normed is not None else ops.cast_rows(x, self.dtype)
        halves = getattr(self.mixer, "forward_halves", None)
        if halves is not None:
            y, rest = halves(h, ctx, cache, write_cache)
            x, h = self.mixer_norm.add_forward(x, y, rest)
        else:
            # a sublayer that offers `forward_for_stream` may hand its last product over as the GEMM's
            # partial sums, which the norm's kernel then adds up itself (nothing runs in between)
            mix = getattr(self.mixer, "forward_for_stream", None)
            y = mix(h, ctx, cache, write_cache) if mix is not None else self.mixer.forward(h, None, ctx, cache, write_cache)
            x, h = self.mixer_norm.add_forward(x, y)
        if self.has_feed_forward:
            ff = getattr(self.feed_forward, "forward_for_stream", None)
            x, h = self.feed_forward_norm.add_forward(x, ff(h, ctx) if ff is not None else self.feed_forward.forward(h, None, ctx))
        if self.token_input is not None:
            x, h = self.token_input.forward(x, h, ctx)
        return x, h


class SandwichNormBlock(PostNormBlock):
    """The arrangement with a norm on each sublayer's input and on its output, over a float32
    residual stream: x <- x + N1b(mixer(N1(x))); x <- x + N2b(ff(N2(x))). The norms are
    `SandwichNorm`s (two gains each). A layer without a feed-forward ends after its first half. The
    kernel that adds a sublayer's normed output also norms the sum for whatever reads it next (the
    feed-forward, or the next block's mixer), so the normed input travels from block to block in
    the place where pre-norm blocks hand it on. Sublayers give their last product as float32 or as
    partial sums (`forward_for_stream`); a feed-forward's `output_bias` joins it before the norm."""

    def forward_chain(self, x: torch.Tensor, normed: torch.Tensor | None, ctx: StepContext, cache: CacheView | None,
                      write_cache: bool, then: Norm | None) -> tuple[torch.Tensor, torch.Tensor | None]:  # fmt: skip
        h = normed if normed is not None else self.mixer_norm.forward(x)
        mix = getattr(self.mixer, "forward_for_stream", None)
        y = mix(h, ctx, cache, write_cache) if mix is not None else self.mixer.forward(h, None, ctx, cache, write_cache)
        if not self.has_feed_forward:
            return self.mixer_norm.add_forward(x, y, then)
        x, h = self.mixer_norm.add_forward(x, y, self.feed_forward_norm)
        ff = getattr(self.feed_forward, "forward_for_stream", None)
        y = ff(h, ctx) if ff is not None else self.feed_forward.forward(h, None, ctx)
        return self.feed_forward_norm.add_forward(x, y, then, getattr(self.feed_forward, "output_bias", None))


class ParallelResidualBlock(PostNormBlock):
    """The arrangement in which mixer and feed-forward read the same float32 stream, each through
    an RMS norm of its own, and are added together: x <- x + mult (mixer(N1 x) + ff(N2 x)); a layer
    without a feed-forward adds the mixer alone. The norms are `RMSNorm`s; `mult` is the mixer
    norm's `mult` (`ScaledRMSNorm`), 1 without one. The kernel that adds a layer's two outputs also
    norms the sum twice for the next block of this kind, so the pair (N1 x, N2 x) travels from
    block to block in the place where pre-norm blocks hand on their normed input. Sublayers give
    float32 outputs (`forward_for_stream` must not leave partial sums: two products are added)."""

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        super().load(tensors)
        self.mult = float(getattr(self.mixer_norm, "mult", 1.0))

    def norms(self) -> tuple[torch.Tensor, torch.Tensor | None, float]:
        return self.mixer_norm.gain, (self.feed_forward_norm.gain if self.has_feed_forward else None), self.mixer_norm.eps

    def forward_chain(self, x: torch.Tensor, normed, ctx: StepContext, cache: CacheView | None,
                      write_cache: bool, then: Norm | None) -> tuple[torch.Tensor, object]:  # fmt: skip
        g1, g2, eps = self.norms()
        if normed is None:
            _, h1, h2 = ops.residual_dual_norm(x, None, None, 1.0, g1, g2, eps, self.dtype, want_stream=False)
        else:
            h1, h2 = normed
        y1 = self.mixer.forward(h1, None, ctx, cache, write_cache)
        y2 = self.feed_forward.forward(h2, None, ctx) if self.has_feed_forward else None
        owner = getattr(then, "block_norms", None) if then is not None else None
        if owner is None:  # the last block, or one of another kind next: the sum alone
            return ops.residual_dual_norm(x, y1, y2, self.mult, None, None, 0.0, self.dtype)[0], None
        n1, n2, eps_next = owner()
        x, h1, h2 = ops.residual_dual_norm(x, y1, y2, self.mult, n1, n2, eps_next, self.dtype)
        return x, (h1, h2)

    def bind_dtype(self, dtype: torch.dtype) -> None:
        super().bind_dtype(dtype)
        self.mixer_norm.block_norms = self.norms  # how the block before this one learns both gains


register_part("block", "parallel_residual", ParallelResidualBlock)
register_part("block", "pre_norm", PreNormBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
register_part("block", "output_norm", OutputNormBlock)
register_part("block", "post_norm", PostNormBlock)
