"""Token embedding (a gather, no scaling, atomserve/model.py:373) and the output head
(float32 logits from the float32 accumulator, atomserve/model.py:388-412; tied to the
embedding when the model says so, atomserve/loader.py:131-138)."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, Part, StateSpec, StepContext, register_part
from atomserve_b200.parts.spec import TensorSpec


class TokenEmbedding(Part):
    def __init__(self, hidden_size: int, prefix: str, vocab_size: int, tensor: str | None = None):
        self.hidden_size, self.vocab_size, self.name = hidden_size, vocab_size, tensor or prefix + "weight"
        self.table: torch.Tensor | None = None
        self.status: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.name]
        # the device's shared status words on a GPU (the engine reads them every step)
        self.status = (ops.status_for(self.table.device).embedding if self.table.is_cuda
                       else torch.zeros(1, dtype=torch.int32))

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(token_ids, self.table, self.status)


class ScaledEmbedding(TokenEmbedding):
    """table[token] * scale as float32: the start of a residual stream that is kept in float32
    whatever the compute dtype."""

    def __init__(self, hidden_size: int, prefix: str, vocab_size: int, scale: float = 1.0, tensor: str | None = None):
        super().__init__(hidden_size, prefix, vocab_size, tensor)
        self.scale = float(scale)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding_scaled(token_ids, self.table, self.scale, self.status)


class NormedEmbedding(TokenEmbedding):
    """RMS norm of table[token] with a gain (`norm_tensor`), as float32: the start of a residual
    stream that is kept in float32 whatever the compute dtype."""

    def __init__(self, hidden_size: int, prefix: str, vocab_size: int, eps: float, tensor: str | None = None,
                 norm_tensor: str | None = None):  # fmt: skip
        super().__init__(hidden_size, prefix, vocab_size, tensor)
        self.eps, self.norm_name = float(eps), norm_tensor or prefix + "norm"
        self.gain: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return super().tensor_specs() + [TensorSpec(self.norm_name, (self.hidden_size,), kind="gain", init="gain")]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        super().load(tensors)
        self.gain = tensors[self.norm_name]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        rows = ops.embedding_scaled(token_ids, self.table, 1.0, self.status)
        return ops.scaled_add_rms_norm(rows, None, 1.0, self.gain, self.eps, torch.float32)[0]


class PairHashEmbedding(TokenEmbedding):
    """table[token] + pairs[(previous token * mul_prev + token * mul_cur) mod buckets] as float32:
    a hashed table of token pairs beside the token table. `pairs` has buckets + 1 rows; the last
    one serves a sequence's first token, which has no predecessor. The token before a step's first
    one is kept per request as state (`last`: that id plus one, 0 after admission), so prompts may
    be cut anywhere and decoded tokens know their predecessor without the host's help."""

    state_in_graphs = True  # one int per request, saved and put back around a capture's warm-up run

    def __init__(self, hidden_size: int, prefix: str, vocab_size: int, buckets: int, mul_prev: int, mul_cur: int,
                 tensor: str | None = None, pair_tensor: str | None = None):  # fmt: skip
        super().__init__(hidden_size, prefix, vocab_size, tensor)
        if buckets < 1:
            raise ValueError(f"a pair table needs at least one bucket, got {buckets}")
        # (a x) mod b = ((a mod b) x) mod b: the multipliers go to the kernel reduced, whatever their size
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev) % int(buckets), int(mul_cur) % int(buckets)
        self.pair_name = pair_tensor or prefix + "pairs"
        self.pairs: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return super().tensor_specs() + [TensorSpec(self.pair_name, (self.buckets + 1, self.hidden_size))]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        super().load(tensors)
        self.pairs = tensors[self.pair_name]

    def state_specs(self) -> list[StateSpec]:
        return [StateSpec("last", (1,), torch.int32)]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise RuntimeError("a pair embedding needs the step's requests and their state: forward_step(ctx, cache)")

    def forward_step(self, ctx: StepContext, cache: CacheView | None) -> torch.Tensor:
        if cache is None or "last" not in cache.state:
            raise RuntimeError("a pair embedding needs its per-request state")
        return ops.pair_embedding(ctx.token_ids, ctx.positions, ctx.req_q_start, ctx.state_slots, cache.state["last"],
                                  self.table, self.pairs, self.mul_prev, self.mul_cur, self.status)  # fmt: skip


class LMHead(Part):
    """`softcap`: logits <- softcap tanh(logits / softcap), on the float32 logits."""

    def __init__(self, hidden_size: int, prefix: str, vocab_size: int, tied: bool, tensor: str | None = None,
                 softcap: float | None = None):  # fmt: skip
        self.hidden_size, self.vocab_size, self.tied, self.name = hidden_size, vocab_size, tied, tensor or prefix + "weight"
        self.softcap = float(softcap) if softcap else None
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [] if self.tied else [TensorSpec(self.name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = tensors[self.name]

    def tie(self, embedding: TokenEmbedding) -> None:
        self.weight = embedding.table

    def forward(self, hidden: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        logits = ops.linear(hidden, self.weight, out_dtype=torch.float32, out=out)
        return ops.softcap_(logits, self.softcap) if self.softcap else logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "scaled_embedding", ScaledEmbedding)
register_part("embedding", "normed_embedding", NormedEmbedding)
register_part("embedding", "pair_hash_embedding", PairHashEmbedding)
register_part("head", "lm_head", LMHead)
