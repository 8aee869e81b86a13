"""SwiGLU feed-forward: residual += W_down (silu(W_gate x) * (W_up x)).

(crates/model/recipes/src/decoder.rs:467-502; silu(z) = z * sigmoid(z) with the
two-branch sigmoid of crates/testing/cpu/reference-ops/src/kernels.rs:12-22.)  The gate
and up matrices are concatenated at load into one [2 I, H] matrix so one GEMM produces
both.  On the bfloat16 path, when I is a multiple of 64, their rows are interleaved in
blocks of 64 (64 gate rows, then the 64 up rows of the same features) and the product
silu(gate) * up is taken in the GEMM's epilogue, so the [T, 2 I] intermediate is never
written (the reference pairs the two projections in one launch and multiplies in a second:
crates/backend/cuda-kernels/src/tile/projection/prefill_gemm_kernels.rs:11-69,
tile/mlp/mlp_kernels.rs:27-36); otherwise the product is a kernel of its own.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.decl import WeightDecl
from .base import FeedForward
from .linear import linear
from .registry import register


class SwiGLU(FeedForward):
    graph_safe = True
    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        for role, name in spec.get("names", ()):            # a description may name the tensors otherwise
            if role not in names:
                raise ValueError(f"swiglu has no tensor role {role!r}")
            names[role] = name
        self.names = {k: prefix + v for k, v in names.items()}
        # what the gate passes through: "silu" (SwiGLU) or "relu"; or a PartSpec of kind "clamped_glu" (limit, sharpness,
        # up_offset): a(min(gate, limit)) * (clamp(up, -limit, limit) + up_offset) with a(g) = g * sigmoid(sharpness * g)
        act = spec.get("activation", "silu")
        self.glu = None
        if isinstance(act, PartSpec):
            if act.kind != "clamped_glu":
                raise ValueError(f"gated feed-forward: unknown activation {act.kind!r}")
            self.glu = (float(act["limit"]), float(act.get("sharpness", 1.0)), float(act.get("up_offset", 0.0)))
            if self.glu[0] <= 0:
                raise ValueError("clamped_glu: limit must be positive")
            act = "silu"
        self.activation = str(act)
        if self.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"gated feed-forward: unknown activation {self.activation!r}")
        self.w_gate_up = self.w_down = None
        self.fused = False

    def declare_weights(self) -> List[WeightDecl]:
        n = self.names
        return [WeightDecl(n["gate"], (self.inter, self.hidden)),
                WeightDecl(n["up"], (self.inter, self.hidden)),
                WeightDecl(n["down"], (self.hidden, self.inter))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        gate, up = tensors[n["gate"]], tensors[n["up"]]
        self.fused = self._fusable(gate.dtype)
        if self.fused:
            blocks = self.inter // 64
            self.w_gate_up = torch.stack(
                [gate.view(blocks, 64, self.hidden), up.view(blocks, 64, self.hidden)], dim=1
            ).reshape(2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[n["down"]].contiguous()

    def _fusable(self, dtype: torch.dtype) -> bool:
        """Whether the gated unit is taken in the tensor-core product's epilogue (gate and up rows interleaved)."""
        return dtype == torch.bfloat16 and self.inter % 64 == 0 and self.hidden % 8 == 0

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        fused = self._fusable(self.ctx.dtype)
        return tokens * self.inter * size * (1 if fused else 3)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step, accumulate: bool = True) -> None:
        """residual += the feed-forward of x (with `accumulate` False: residual = it)."""
        T = x.shape[0]
        ws, dt = self.ctx.workspace, self.ctx.dtype
        act = ws.buffer("mlp.act", (T, self.inter), dt)
        ops.scope("feed_forward.gate_up (gate inside)" if self.fused else "feed_forward.gate_up")
        if self.fused and ops.gemm_tc_eligible(x, self.w_gate_up, act):
            ops.gemm_tc(x, self.w_gate_up, act, swiglu=True, gate=self.activation, glu=self.glu)
        elif self.fused:
            raise ops.KernelError("SwiGLU: the interleaved weight needs the tensor-core GEMM, which refused this input")
        else:
            gate_up = ws.buffer("mlp.gate_up", (T, 2 * self.inter), dt)
            linear(x, self.w_gate_up, gate_up)
            ops.scope("feed_forward.swiglu")
            if self.glu is not None:
                ops.glu_mul(gate_up, act, *self.glu)
            else:
                ops.silu_mul(gate_up, act, self.activation)
        ops.scope("feed_forward.down")
        linear(act, self.w_down, residual, accumulate=accumulate)


class NoFeedForward(FeedForward):
    """A layer that has only its mixer: blocks skip the feed-forward's norm and sublayer."""
    graph_safe = True
    absent = True

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step) -> None:
        return None


register("feed_forward", "swiglu", SwiGLU)
register("feed_forward", "none", NoFeedForward)
