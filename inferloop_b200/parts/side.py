"""A sublayer fed by the token itself (feed-forward kind `token_gated`).

Every token has a row in a second table; layer i owns the columns [i * dim, (i + 1) * dim) of it:

    e = S[token][col0 : col0 + dim];   out = P (gelu_tanh(G x) * e)        G [dim, hidden], P [hidden, dim]

The table belongs to the model (every layer declares the same tensor and reads its own slice).  The
gate's product and the output's are the engine's products; the gate itself is one element-wise kernel
that also looks the token's row up.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from .base import FeedForward
from .linear import linear
from .registry import register


class TokenGatedSide(FeedForward):
    graph_safe = True

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.dim = int(spec["dim"])
        self.col0 = int(spec["column"])
        self.vocab = int(spec["vocab_size"])
        self.table_width = int(spec["table_width"])
        if self.col0 < 0 or self.col0 + self.dim > self.table_width:
            raise ValueError(f"token_gated: columns {self.col0} .. {self.col0 + self.dim} lie outside a table of {self.table_width}")
        self.table_name = str(spec["table"])                      # a name of the model, not under the layer's prefix
        self.gate_name = prefix + str(spec.get("gate", "gate"))
        self.proj_name = prefix + str(spec.get("proj", "proj"))
        self.table = self.w_gate = self.w_proj = None

    def declare_weights(self) -> List[WeightDecl]:
        return [WeightDecl(self.table_name, (self.vocab, self.table_width), role="table"),
                WeightDecl(self.gate_name, (self.dim, self.hidden)), WeightDecl(self.proj_name, (self.hidden, self.dim))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.table_name]
        if not self.table.is_contiguous():
            self.table = self.table.contiguous()
        self.w_gate = tensors[self.gate_name].contiguous()
        self.w_proj = tensors[self.proj_name].contiguous()

    def scratch_bytes(self, tokens: int) -> int:
        return 2 * tokens * self.dim * torch.empty((), dtype=self.ctx.dtype).element_size()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step) -> None:
        T, ws, dt = x.shape[0], self.ctx.workspace, self.ctx.dtype
        a = ws.buffer("side.gate", (T, self.dim), dt)
        ops.scope("token_side.gate")
        linear(x, self.w_gate, a)
        g = ws.buffer("side.gated", (T, self.dim), dt)
        ops.gated_rows(a, self.table, self.col0, step.tokens, g)
        ops.scope("token_side.projection")
        linear(g, self.w_proj, residual, accumulate=True)


register("feed_forward", "token_gated", TokenGatedSide)
