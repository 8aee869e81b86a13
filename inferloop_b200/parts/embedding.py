"""Parts that turn token ids into the first residual stream (role `embedding`).

`hashed_pairs`: the token's row of the token table plus a row of a second, hashed table that is
chosen by the pair (previous token, token):

    x_t = E[tok_t] + P[(tok_{t-1} * mul_prev + tok_t * mul_cur) mod buckets],   P[buckets] for a sequence's first token

followed, when the spec names a norm, by that norm (an RMS norm: fused into the same kernel).  The
token before a step's first token is state of the request: one int32 per state slot, written after
every step.  With `keep`, the rows are also left in the workspace buffer of that name, [tokens,
hidden] 32-bit, for blocks that read the embedding's output later.  `buckets` 0: no second table.

`normed`: the token's row of the token table (times `scale`, default 1), then the norm the spec names (any norm
that can write over its own input: an element-wise one).
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from . import registry
from .base import CacheNeeds, Embedding, SlotStateNeed
from .norm import RMSNorm


class HashedPairsEmbedding(Embedding):
    graph_safe = True

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.buckets = int(spec.get("buckets", 0))
        self.mul_prev = int(spec.get("mul_prev", 0))
        self.mul_cur = int(spec.get("mul_cur", 0))
        self.table_name = prefix + str(spec.get("table", "pairs"))
        self.keep = spec.get("keep")
        self.norm = None
        if spec.get("norm") is not None:
            self.norm = registry.build_norm(spec["norm"], ctx, prefix + str(spec.get("norm_name", "embed_norm.")), width=self.hidden)
            if not isinstance(self.norm, RMSNorm):
                raise ValueError("hashed_pairs: the norm after the embedding must be an RMS norm")
        self.pairs = None

    def declare_weights(self) -> List[WeightDecl]:
        out = [WeightDecl(self.table_name, (self.buckets + 1, self.hidden), role="table")] if self.buckets else []
        return out + (self.norm.declare_weights() if self.norm is not None else [])

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        if self.buckets:
            self.pairs = tensors[self.table_name].contiguous()
        if self.norm is not None:
            self.norm.bind(tensors)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(slots=(SlotStateNeed("previous_token", (), torch.int32),) if self.buckets else ())

    def scratch_bytes(self, tokens: int) -> int:
        return tokens * self.hidden * 4 if self.keep else 0

    def forward(self, step, table: torch.Tensor, hidden: torch.Tensor, state: Mapping[str, torch.Tensor]) -> None:
        keep = None
        if self.keep:
            keep = self.ctx.workspace.buffer(str(self.keep), hidden.shape, torch.float32)
        prev = state.get("previous_token") if self.buckets else None
        if self.buckets and prev is None:
            raise ops.KernelError("hashed_pairs: the previous tokens' state slots are missing")
        ops.embed_pairs(step, table, self.pairs, self.buckets, self.mul_prev, self.mul_cur, prev,
                        self.norm.weight if self.norm is not None else None, self.norm.eps if self.norm is not None else 0.0,
                        hidden, keep)
        if prev is not None:
            ops.store_last_tokens(step, prev)


class NormedEmbedding(Embedding):
    graph_safe = True
    """spec: hidden_size, norm (a PartSpec of role norm), norm_name (the norm's tensor prefix), scale (default 1)."""

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.scale = float(spec.get("scale", 1.0))
        self.norm = registry.build_norm(spec["norm"], ctx, prefix + str(spec.get("norm_name", "embed_norm.")), width=self.hidden)
        if not getattr(self.norm, "graph_safe", False):
            raise ValueError("normed embedding: the norm must read the batch from device memory alone")

    def declare_weights(self) -> List[WeightDecl]:
        return self.norm.declare_weights()

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.norm.bind(tensors)

    def forward(self, step, table: torch.Tensor, hidden: torch.Tensor, state: Mapping[str, torch.Tensor]) -> None:
        ops.embed(step.tokens, table, hidden, self.scale, 1)
        self.norm.forward(hidden, hidden)


registry.register("embedding", "hashed_pairs", HashedPairsEmbedding)
registry.register("embedding", "normed", NormedEmbedding)
