"""RMSNorm: x / sqrt(mean(x^2) + eps) * weight, computed in 32-bit
(crates/testing/cpu/reference-ops/src/kernels.rs:38-54; weight offset 0 for this family,
crates/model/package/src/providers/qwen/mod.rs:252).  With `groups` = n the row is cut into n equal
consecutive parts and each part is divided by its own root mean square (one weight over the whole row)."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from .base import Norm
from .registry import register


class RMSNorm(Norm):
    graph_safe = True
    """spec: eps; optional `weight_suffix` (default "weight"): the weight is the tensor
    prefix + suffix, of the width that the owner gives; optional `offset` (default 0): the
    stored tensor is the weight minus this constant (a weight kept around zero: offset 1);
    optional `groups` (default 1): parts of the row that are normed each by itself."""

    def __init__(self, spec, ctx, prefix: str = "", width: int = 0, name: str = "weight") -> None:
        super().__init__(spec, ctx, prefix)
        self.eps = float(spec["eps"])
        self.width = int(width or spec.get("width", 0))
        self.weight_name = prefix + str(spec.get("weight_suffix", name))
        self.offset = float(spec.get("offset", 0.0))
        self.groups = int(spec.get("groups", 1))
        if self.groups < 1 or (self.width and self.width % self.groups):
            raise ValueError(f"a norm over {self.width} elements cannot be cut into {self.groups} equal parts")
        self.weight = None

    def declare_weights(self) -> List[WeightDecl]:
        return [WeightDecl(self.weight_name, (self.width,), role="vector", init="around_zero" if self.offset else "norm")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()      # 32-bit: the sum a norm in 32-bit would form

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        if self.groups > 1:
            ops.group_norm_add(x, self.weight, self.eps, self.groups, out=out)
        else:
            ops.rmsnorm(x, self.weight, self.eps, out)


register("norm", "rms", RMSNorm)
