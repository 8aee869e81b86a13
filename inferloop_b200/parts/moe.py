"""Routed feed-forward: every token runs `top_k` of `experts` small SwiGLU feed-forwards.

  z = W_router x                (32-bit; x may be the compute dtype's rounding)
  s = sigmoid(z)  or  softmax(z) over the experts          (`score`)
  (`router_bias`: z = W_router x + b)
  the top_k experts with the largest s (ties to the lower index), weights w = their s,
  divided by their sum when `renormalize` (softmax + renormalize = the softmax over the chosen logits alone)
  y = sum_j expert_j(w_j x)     (`weight_on` = "input")   or   sum_j w_j expert_j(x)   ("output")
  y += sigmoid(W_gate x) * shared(x)    when the description has a shared expert (`shared_inter`;
  `shared_gate` False leaves the multiplier out)
  (`correction`: the experts are ranked by s + c with a stored vector c, the weights stay s;  `groups` = (count, keep):
  the experts form `count` equal groups of neighbours, a group ranks by its best member, and only experts of the best
  `keep` groups can be chosen;  `renorm_eps` joins the sum that `renormalize` divides by;  `route_scale` multiplies the weights)

The experts' matrices are stacked at load into [experts, 2 I, H] (gate rows, then up rows) and
[experts, H, I].  A step sorts its (token, choice) pairs by expert on the device into rows
padded so that a block of rows belongs to one expert (csrc/moe.cu), gathers the inputs into
that order, runs the two grouped products over it, and adds each token's rows back in choice
order together with the shared expert.  No size depends on the routing, so decode steps can
be replayed as recorded graphs.  On the bfloat16 path, when I is a multiple of 64, the grouped
products run on the tcgen05 tensor cores in blocks of 128 or 256 rows (csrc/moe_gemm_tcgen05.cu) with
gate and up rows interleaved in blocks of 64 and silu(gate) * up taken in the first product's
epilogue, as the dense feed-forward does; otherwise they are the exact product in blocks of 16.
The router's and the gate's logits come from one 32-bit product over the rows [W_router; W_gate]
(a warp per token: the matrix has few rows).
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.decl import WeightDecl
from .base import FeedForward
from .mlp import SwiGLU
from .registry import register


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.experts = int(spec["experts"])
        self.top = int(spec["top_k"])
        self.inter = int(spec["expert_inter"])
        self.score = str(spec.get("score", "softmax"))
        self.renormalize = bool(spec.get("renormalize", False))
        self.weight_on = str(spec.get("weight_on", "output"))
        self.router_bias = bool(spec.get("router_bias", False))       # a vector added to the router's logits
        self.correction = bool(spec.get("correction", False))         # a vector added to the scores for the ranking alone
        groups = spec.get("groups")
        self.groups, self.keep = (int(groups[0]), int(groups[1])) if groups else (1, 1)
        self.route_scale = float(spec.get("route_scale", 1.0))
        self.renorm_eps = float(spec.get("renorm_eps", 0.0))
        if self.groups < 1 or self.experts % self.groups or not 1 <= self.keep <= self.groups or self.groups > 32:
            raise ValueError(f"routed feed-forward: {self.groups} groups (keeping {self.keep}) of {self.experts} experts")
        if self.top > self.experts // self.groups * self.keep:
            raise ValueError(f"routed feed-forward: top {self.top} exceeds the experts of the {self.keep} kept groups")
        # the experts' gated unit: a(gate) * (up + up_offset), a(g) = g * sigmoid(sharpness * g); kind "clamped_glu" also
        # takes min(gate, limit) and clamp(up, -limit, limit) first.  (limit, sharpness, up_offset); the default is SwiGLU.
        act = spec.get("activation")
        if act is None or act.kind == "swiglu":
            self.act = (0.0, 1.0, 0.0)
        elif act.kind == "clamped_glu":
            self.act = (float(act["limit"]), float(act.get("sharpness", 1.0)), float(act.get("up_offset", 0.0)))
            if self.act[0] <= 0:
                raise ValueError("clamped_glu: limit must be positive")
        else:
            raise ValueError(f"the experts' activation must be 'swiglu' or 'clamped_glu', found {act.kind!r}")
        self.shared_inter = int(spec.get("shared_inter") or 0)
        self.shared_gate = bool(spec.get("shared_gate", False)) and self.shared_inter > 0
        if self.score not in ("sigmoid", "softmax"):
            raise ValueError(f"router score must be 'sigmoid' or 'softmax', found {self.score!r}")
        if self.weight_on not in ("input", "output"):
            raise ValueError(f"weight_on must be 'input' or 'output', found {self.weight_on!r}")
        if not 0 < self.top <= self.experts:
            raise ValueError(f"top_k {self.top} of {self.experts} experts")
        # tensor names under the prefix: {e} is the expert's number
        names = {"router": "router.weight", "router_bias": "router.bias", "correction": "router.correction", "gate": "experts.{e}.gate_proj.weight", "up": "experts.{e}.up_proj.weight",
                 "down": "experts.{e}.down_proj.weight", "shared_gate": "shared_expert_gate.weight",
                 "shared_prefix": "shared_expert."}
        for role, name in spec.get("names", ()):
            if role not in names:
                raise ValueError(f"routed feed-forward has no tensor role {role!r}")
            names[role] = name
        self.names = {k: prefix + v for k, v in names.items()}
        self.shared = None
        if self.shared_inter:
            self.shared = SwiGLU(PartSpec.make("swiglu", hidden_size=self.hidden, intermediate_size=self.shared_inter,
                                               names=tuple(spec.get("shared_names", ()))), ctx, self.names["shared_prefix"])
        self.w_router = self.w_gate_up = self.w_down = self.b_router = self.c_router = None
        self.fused = False          # gate/up rows interleaved for the tensor-core product's SwiGLU epilogue

    # ------------------------------------------------------------------ weights
    def declare_weights(self) -> List[WeightDecl]:
        n, H, I = self.names, self.hidden, self.inter
        out = [WeightDecl(n["router"], (self.experts, H))]
        if self.router_bias:
            out.append(WeightDecl(n["router_bias"], (self.experts,), "vector", "bias"))
        if self.correction:
            out.append(WeightDecl(n["correction"], (self.experts,), "vector", "bias"))
        for e in range(self.experts):
            out += [WeightDecl(n["gate"].format(e=e), (I, H)), WeightDecl(n["up"].format(e=e), (I, H)),
                    WeightDecl(n["down"].format(e=e), (H, I))]
        if self.shared is not None:
            out += self.shared.declare_weights()
        if self.shared_gate:
            out.append(WeightDecl(n["shared_gate"], (1, H)))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        rows = [tensors[n["router"]]] + ([tensors[n["shared_gate"]]] if self.shared_gate else [])
        self.w_router = torch.cat(rows, dim=0).contiguous()
        if self.router_bias:
            self.b_router = tensors[n["router_bias"]].contiguous()
        if self.correction:
            self.c_router = tensors[n["correction"]].contiguous()
        gates = [tensors[n["gate"].format(e=e)] for e in range(self.experts)]
        ups = [tensors[n["up"].format(e=e)] for e in range(self.experts)]
        self.fused = gates[0].dtype == torch.bfloat16 and self.inter % 64 == 0 and self.hidden % 8 == 0
        if self.fused:
            blocks = self.inter // 64
            self.w_gate_up = torch.stack([
                torch.stack([g.view(blocks, 64, self.hidden), u.view(blocks, 64, self.hidden)], dim=1).reshape(2 * self.inter, self.hidden)
                for g, u in zip(gates, ups)]).contiguous()
        else:
            self.w_gate_up = torch.stack([torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]).contiguous()
        self.w_down = torch.stack([tensors[n["down"].format(e=e)] for e in range(self.experts)]).contiguous()
        if self.shared is not None:
            self.shared.bind(tensors)

    def _block_rows(self, tokens: int) -> int:
        """Rows of a block of the sorted order: the exact product's 16, or the tensor-core
        product's tile height: 128 rows (256 only when `ops.MOE_WIDE_BLOCKS` is set: measured slower than
        persistent CTAs over 128-row tiles at every size tried)."""
        fused = self.ctx.dtype == torch.bfloat16 and self.inter % 64 == 0 and self.hidden % 8 == 0
        if not fused:
            return ops.GROUP_ROWS_SIMT
        wide = ops.MOE_WIDE_BLOCKS and tokens * self.top >= self.experts * 4 * ops.GROUP_ROWS_TC_WIDE
        return ops.GROUP_ROWS_TC_WIDE if wide else ops.GROUP_ROWS_TC

    def _rows(self, tokens: int) -> int:
        return ops.moe_plan_rows(tokens * self.top, self.experts, self._block_rows(tokens))

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        rows = self._rows(tokens)
        own = rows * ((self.hidden + 3 * self.inter) * size + self.hidden * 4) + tokens * (self.experts + 1 + 3 * self.top) * 4 + rows * 4
        shared = (self.shared.scratch_bytes(tokens) + tokens * self.hidden * 4) if self.shared is not None else 0
        return own + shared

    # ------------------------------------------------------------------ run
    def forward(self, x: torch.Tensor, residual: torch.Tensor, step) -> None:
        T, H, I, E, K = x.shape[0], self.hidden, self.inter, self.experts, self.top
        ws, dt = self.ctx.workspace, self.ctx.dtype
        block = self._block_rows(T)
        rows = self._rows(T)
        ops.scope("feed_forward.router")
        logits = ws.buffer("moe.logits", (T, self.w_router.shape[0]), torch.float32)
        ops.moe_logits(x, self.w_router, logits)
        choice = ws.buffer("moe.choice", (T * K,), torch.int32)
        weight = ws.buffer("moe.weight", (T * K,), torch.float32)
        ops.moe_route(logits, E, K, self.score == "softmax", self.renormalize, choice, weight, bias=self.b_router,
                      correction=self.c_router, groups=self.groups, keep=self.keep, scale=self.route_scale, renorm_eps=self.renorm_eps)
        pos = ws.buffer("moe.pos", (T * K,), torch.int32)
        block_expert = ws.buffer("moe.block_expert", (rows // block,), torch.int32)
        ops.moe_plan(choice, E, block, pos, block_expert)
        ops.scope("feed_forward.experts")
        a = ws.buffer("moe.rows", (rows, H), dt)
        ops.moe_gather(x, weight if self.weight_on == "input" else None, pos, K, a)
        act = ws.buffer("moe.act", (rows, I), dt)
        routed = ws.buffer("moe.routed", (rows, H), torch.float32)
        if self.fused:
            if not (ops.moe_gemm_tc_eligible(a, self.w_gate_up, swiglu=True) and ops.moe_gemm_tc_eligible(act, self.w_down)):
                raise ops.KernelError("routed experts: the interleaved weights need the tensor-core product, which refused this input")
            ops.moe_gemm_tc(a, self.w_gate_up, act, block_expert, swiglu=True, block_rows=block, act=self.act)
            ops.moe_gemm_tc(act, self.w_down, routed, block_expert, block_rows=block)
        else:
            gate_up = ws.buffer("moe.gate_up", (rows, 2 * I), dt)
            ops.gemm_simt_grouped(a, self.w_gate_up, gate_up, block_expert)
            if self.act == (0.0, 1.0, 0.0):
                ops.silu_mul(gate_up, act)
            else:
                ops.glu_mul(gate_up, act, *self.act)
            ops.gemm_simt_grouped(act, self.w_down, routed, block_expert)
        shared_out = None
        if self.shared is not None:
            ops.scope("feed_forward.shared_expert")
            shared_out = ws.buffer("moe.shared", (T, H), torch.float32)
            self.shared.forward(x, shared_out, step, accumulate=False)
        ops.scope("feed_forward.combine")
        ops.moe_combine(routed, pos, weight if self.weight_on == "output" else None, K, shared_out,
                        logits[:, E] if self.shared_gate else None, residual)


register("feed_forward", "routed_experts", RoutedExperts)
