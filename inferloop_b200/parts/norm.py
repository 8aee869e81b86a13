"""RMSNorm: x / sqrt(mean(x^2) + eps) * weight, computed in 32-bit
(crates/testing/cpu/reference-ops/src/kernels.rs:38-54; weight offset 0 for this family,
crates/model/package/src/providers/qwen/mod.rs:252).  With `groups` = n the row is cut into n equal
consecutive parts and each part is divided by its own root mean square (one weight over the whole row).

Dynamic Tanh (`dyt`): tanh(alpha x) * weight + bias, element by element, with one stored scalar alpha: a norm that
takes no mean and no variance, so a row's result does not depend on the rest of the row."""
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


class DynamicTanh(Norm):
    graph_safe = True
    """spec: optional `weight_suffix` (default "weight"), `bias_suffix` (default ".b") and `alpha_suffix` (default
    ".alpha"): the weight is the tensor prefix + weight_suffix, the bias and the scalar are that name + their suffix."""

    def __init__(self, spec, ctx, prefix: str = "", width: int = 0, name: str = "weight") -> None:
        super().__init__(spec, ctx, prefix)
        self.width = int(width or spec.get("width", 0))
        self.weight_name = prefix + str(spec.get("weight_suffix", name))
        self.bias_name = self.weight_name + str(spec.get("bias_suffix", ".b"))
        self.alpha_name = self.weight_name + str(spec.get("alpha_suffix", ".alpha"))
        self.weight = self.bias = self.alpha = None

    def declare_weights(self) -> List[WeightDecl]:
        return [WeightDecl(self.weight_name, (self.width,), role="vector", init="norm"),
                WeightDecl(self.bias_name, (self.width,), role="vector", init="bias"),
                WeightDecl(self.alpha_name, (), role="vector", init="mix")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()
        self.bias = tensors[self.bias_name].contiguous()
        self.alpha = tensors[self.alpha_name].reshape(1).contiguous()

    @property
    def tensors(self):
        """(alpha, weight, bias) as the kernels take them."""
        return (self.alpha, self.weight, self.bias)

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """`out` may be `x` itself: every element depends on its own input alone."""
        ops.dyt(x, self.alpha, self.weight, self.bias, out)


register("norm", "rms", RMSNorm)
register("norm", "dyt", DynamicTanh)
