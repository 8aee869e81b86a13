"""Mixers with a state of fixed size per request, and the mixer that runs several mixers side by side.

`gated_linear_recurrence` (the recurrent block of Griffin with its real-gated linear recurrent unit):

    y = gelu_tanh(W_y h + b_y);  u = causal conv over `taps` tokens, per channel, with bias, of (W_x h + b_x)
    u is cut into `blocks` equal parts; in part b: r = sigmoid(Ra_b u_b + ra_b), i = sigmoid(Ri_b u_b + ri_b)
    a = exp(-rate * r * softplus(lam));   S_t = a S_{t-1} + sqrt(1 - a^2) * i * u_t;   out = W_o (S * y)

State per request: S [width] in 32-bit and the last taps - 1 inputs of the convolution.  The two input
products are one product; the convolution is the state-space layer's (without its activation); the gates'
block-diagonal products run with 32-bit accuracy (per-block products of csrc/latent.cu: on the tensor cores with the
32-bit input cut into three exact bfloat16 pieces when the matrices are bfloat16, else on 32-bit lanes); the gates, the
decay, the recurrence and the output gate are one kernel (csrc/recurrent.cu), chunked for long portions.

`decayed_linear_attention` (lightning attention): q, k, v = silu(W h) per head, S_t = decay_h S_{t-1} + k_t v_t^T,
o_t = S_t^T q_t; the heads together are RMS-normed with a weight, multiplied by sigmoid(W_g h) and by the
constant `out_scale`, and projected.  State per request: S [heads, dim, vdim] in 32-bit.  The recurrence is the
state-space layer's scan with a stored decay and unit step sizes (csrc/ssm.cu, `fixed`), so long portions run in
chunks side by side.

`parallel`: several mixers read the same input and add into the same output, each with its own tensors under its
own prefix, its own cache (at most one of them paged) and its own constant on its output.
"""
from __future__ import annotations

import dataclasses
from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from . import registry
from .base import CacheNeeds, Mixer, SlotStateNeed
from .linear import linear


def _names(defaults: dict, spec, prefix: str, what: str) -> dict:
    names = dict(defaults)
    for role, name in spec.get("names", ()):
        if role not in names:
            raise ValueError(f"{what} has no tensor role {role!r}")
        names[role] = name
    return {k: prefix + v for k, v in names.items()}


class GatedLinearRecurrence(Mixer):
    graph_safe = True

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.width = int(spec["width"])
        self.blocks = int(spec["blocks"])
        self.taps = int(spec["taps"])
        self.rate = float(spec.get("rate", 8.0))
        self.out_scale = float(spec.get("out_scale", 1.0))
        if self.out_scale != 1.0:
            raise ValueError("gated_linear_recurrence: no constant on the output is served")
        if self.blocks < 1 or self.width % self.blocks:
            raise ValueError(f"{self.width} channels cannot be cut into {self.blocks} equal blocks")
        self.block_width = self.width // self.blocks
        self.names = _names({"y": "y", "yb": "y.b", "x": "x", "xb": "x.b", "conv": "conv", "conv_bias": "conv.b", "ra": "ra",
                             "rab": "ra.b", "ri": "ri", "rib": "ri.b", "lam": "lam", "o": "o"}, spec, prefix, "the gated recurrence")
        self.w_in = self.b_in = self.conv_w = self.conv_b = self.w_gates = self.r_bias = self.i_bias = self.lam = self.w_o = None
        self.split = False

    def declare_weights(self) -> List[WeightDecl]:
        n, W, H, B, bw = self.names, self.width, self.hidden, self.blocks, self.block_width
        return [WeightDecl(n["y"], (W, H)), WeightDecl(n["yb"], (W,), "vector", "bias"),
                WeightDecl(n["x"], (W, H)), WeightDecl(n["xb"], (W,), "vector", "bias"),
                WeightDecl(n["conv"], (W, self.taps), "vector", "mix"), WeightDecl(n["conv_bias"], (W,), "vector", "bias"),
                WeightDecl(n["ra"], (B, bw, bw)), WeightDecl(n["rab"], (B, bw), "vector", "bias"),
                WeightDecl(n["ri"], (B, bw, bw)), WeightDecl(n["rib"], (B, bw), "vector", "bias"),
                WeightDecl(n["lam"], (W,), "vector", "around_zero"), WeightDecl(n["o"], (H, W))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n["y"]], tensors[n["x"]]], dim=0).contiguous()          # one product gives y | x
        self.b_in = torch.cat([tensors[n["yb"]], tensors[n["xb"]]]).contiguous()
        self.conv_w = tensors[n["conv"]].contiguous()
        self.conv_b = tensors[n["conv_bias"]].contiguous()
        # a block's two gate matrices side by side, [blocks, in, 2 out].  The gates are 32-bit arithmetic: bfloat16 matrices
        # take the tensor-core product whose 32-bit input is cut into three exact pieces, others the 32-bit lanes
        ra, ri = tensors[n["ra"]], tensors[n["ri"]]
        self.w_gates = torch.cat([ra.transpose(1, 2), ri.transpose(1, 2)], dim=2).contiguous()
        self.split = ra.dtype == torch.bfloat16 and ops.head_matmul_split_supported(self.block_width, 2 * self.block_width, self.width, 2 * self.width)
        if not self.split:
            self.w_gates = self.w_gates.float()
        self.r_bias = tensors[n["rab"]].reshape(-1).contiguous()
        self.i_bias = tensors[n["rib"]].reshape(-1).contiguous()
        self.lam = tensors[n["lam"]].contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(slots=(SlotStateNeed("state", (self.width,), torch.float32),
                                 SlotStateNeed("conv", (max(self.taps - 1, 0), self.width), torch.float32)))

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        chunks = -(-tokens // ops.LRU_CHUNK) + 1
        return tokens * self.width * (3 * size + 3 * 4) + 2 * chunks * self.width * 4

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        T, W, ws, dt = x.shape[0], self.width, self.ctx.workspace, self.ctx.dtype
        proj = ws.buffer("lru.proj", (T, 2 * W), dt)
        ops.scope("recurrence.in_projection")
        linear(x, self.w_in, proj, self.b_in)
        ops.scope("recurrence.convolution")
        u = ws.buffer("lru.u", (T, W), torch.float32)
        ops.ssm_conv(proj, W, W, self.conv_w, self.conv_b, cache.state["conv"], step, u, activation="none")
        ops.scope("recurrence.gates")
        gates = ws.buffer("lru.gates", (T, 2 * W), torch.float32)
        if self.split:
            ops.head_matmul_split(u, self.w_gates, gates)
        else:
            ops.head_matmul(u, self.w_gates, gates)
        ops.scope("recurrence.scan")
        gated = ws.buffer("lru.gated", (T, W), dt)
        ops.lru_scan(gates, u, proj, 0, self.r_bias, self.i_bias, self.lam, self.rate, cache.state["state"], gated, step,
                     self.block_width, workspace=ws)
        ops.scope("recurrence.out_projection")
        linear(gated, self.w_o, residual, accumulate=True)


class DecayedLinearAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec["v_head_dim"])
        self.decay = tuple(float(v) for v in spec["decay"])
        self.eps = float(spec["eps"])
        self.out_scale = float(spec.get("out_scale", 1.0))
        if len(self.decay) != self.heads or any(not 0.0 <= v <= 1.0 for v in self.decay):
            raise ValueError(f"decayed_linear_attention: {self.heads} heads need as many decays in [0, 1], found {self.decay}")
        self.inner = self.heads * self.dv
        self.channels = self.inner + 2 * self.heads * self.d           # v | k | q: what the recurrence reads
        self.names = _names({"q": "q", "k": "k", "v": "v", "g": "g", "norm": "norm", "o": "o"}, spec, prefix, "the linear attention")
        self.w_in = self.norm_w = self.w_o = self.decays = None

    def declare_weights(self) -> List[WeightDecl]:
        n, H = self.names, self.hidden
        return [WeightDecl(n["q"], (self.heads * self.d, H)), WeightDecl(n["k"], (self.heads * self.d, H)),
                WeightDecl(n["v"], (self.inner, H)), WeightDecl(n["g"], (self.inner, H)),
                WeightDecl(n["norm"], (self.inner,), "vector", "norm"), WeightDecl(n["o"], (H, self.inner))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        # one product gives v | k | q | g: the recurrence reads values, keys and queries in that order
        self.w_in = torch.cat([tensors[n["v"]], tensors[n["k"]], tensors[n["q"]], tensors[n["g"]]], dim=0).contiguous()
        self.norm_w = tensors[n["norm"]].contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.decays = torch.tensor(self.decay, dtype=torch.float32, device=self.w_o.device)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(slots=(SlotStateNeed("state", (self.heads, self.d, self.dv), torch.float32),))

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        chunks = -(-tokens // ops.SSM_CHUNK) + 1
        return (tokens * ((self.channels + 2 * self.inner) * size + (self.channels + self.inner) * 4)
                + chunks * self.heads * (self.d * self.dv + 1) * 4)

    def input_rows(self):
        """(matrix, bias or None) of the one product this mixer starts with (see `forward_projected`)."""
        return self.w_in, None

    def take_input_rows(self, rows: torch.Tensor) -> None:
        """The same matrix as a view of the stacked one: no second copy is kept."""
        self.w_in = rows

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        T, ws, dt = x.shape[0], self.ctx.workspace, self.ctx.dtype
        proj = ws.buffer("linattn.proj", (T, self.channels + self.inner), dt)
        ops.scope("linear_attention.in_projection")
        linear(x, self.w_in, proj)
        self.forward_projected(proj, residual, step, cache)

    def output_rows(self):
        """(matrix [hidden, heads * v_head_dim], bias or None) of the product this mixer ends with."""
        return self.w_o, None

    def forward_projected(self, proj: torch.Tensor, residual: torch.Tensor, step, cache, out=None) -> None:
        """The mixer from its projection's output on: `proj` [T, v | k | q | gate], rows of any stride.  With `out`
        [T, heads * v_head_dim] (rows of any stride) the normed, gated rows go there and the output product is left to the caller."""
        T, ws, dt = proj.shape[0], self.ctx.workspace, self.ctx.dtype
        ops.scope("linear_attention.activation")
        act = ws.buffer("linattn.act", (T, self.channels), torch.float32)
        ops.silu_rows(proj, self.channels, act)
        ops.scope("linear_attention.scan")
        y = ws.buffer("linattn.y", (T, self.inner), torch.float32)
        ops.ssm_scan(act, None, 0, None, self.decays, None, cache.state["state"], y, step, self.heads, self.dv, self.d, self.heads,
                     workspace=ws, fixed_decay=True)
        ops.scope("linear_attention.norm_gate")
        gated = out if out is not None else ws.buffer("linattn.gated", (T, self.inner), dt)
        ops.rms_gate(y, proj[:, self.channels:], self.norm_w, self.eps, gated, self.out_scale)
        if out is None:
            ops.scope("linear_attention.out_projection")
            linear(gated, self.w_o, residual, accumulate=True)


class ParallelMixers(Mixer):
    """spec: `branches` = ((sub-prefix, PartSpec of role mixer), ...).  Every branch reads the block's input and adds
    into the block's output; a branch's constant on its output is its own parameter (`out_scale`).  Branches that start
    with one product of the input each (`input_rows` / `forward_projected`) share ONE product: their matrices are
    stacked at load (each branch keeps a view of its rows) and every branch reads its columns of the result.  Branches
    that also end with one product each (`output_rows`) share that too: every branch writes what its product would read
    into its columns of one matrix, and one product with the branches' matrices side by side adds all of them into the
    block's output (the sum over a row of the stacked matrix is the sum of the branches' products)."""

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        branches = tuple(spec["branches"])
        if not branches:
            raise ValueError("parallel: no branches")
        self.parts = [registry.build("mixer", part, ctx, prefix + sub) for sub, part in branches]
        self.w_all = self.b_all = self.w_out = self.b_out = None
        self.columns, self.out_columns = [], []
        if sum(1 for p in self.parts if p.cache_needs().paged is not None) > 1:
            raise ValueError("parallel: at most one branch may keep keys and values in pages")

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in self.parts)

    def declare_weights(self) -> List[WeightDecl]:
        return [d for p in self.parts for d in p.declare_weights()]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self.parts:
            p.bind(tensors)
        self.w_all = self.b_all = self.w_out = self.b_out = None
        self.columns, self.out_columns = [], []
        if len(self.parts) < 2 or not all(hasattr(p, "input_rows") and hasattr(p, "forward_projected") for p in self.parts):
            return
        rows = [p.input_rows() for p in self.parts]
        # every branch's columns start on a 16-byte boundary of the shared result
        if any(w.shape[0] % 8 for w, _ in rows) or len({(w.dtype, w.shape[1]) for w, _ in rows}) != 1:
            return
        self.w_all = torch.cat([w for w, _ in rows], dim=0).contiguous()
        if any(b is not None for _, b in rows):
            self.b_all = torch.cat([b if b is not None else torch.zeros(w.shape[0], dtype=torch.float32, device=w.device)
                                    for w, b in rows]).contiguous()
        at = 0
        for p, (w, _) in zip(self.parts, rows):
            self.columns.append((at, at + w.shape[0]))
            if hasattr(p, "take_input_rows"):
                p.take_input_rows(self.w_all[at:at + w.shape[0]])
            at += w.shape[0]
        outs = [p.output_rows() if hasattr(p, "output_rows") else None for p in self.parts]
        if any(o is None for o in outs) or any(w.shape[1] % 8 for w, _ in outs) or len({(w.dtype, w.shape[0]) for w, _ in outs}) != 1:
            return
        self.w_out = torch.cat([w for w, _ in outs], dim=1).contiguous()
        biases = [b for _, b in outs if b is not None]
        self.b_out = torch.stack(biases).sum(0).contiguous() if biases else None
        at = 0
        for w, _ in outs:
            self.out_columns.append((at, at + w.shape[1]))
            at += w.shape[1]

    def cache_needs(self) -> CacheNeeds:
        paged, slots = None, []
        for i, p in enumerate(self.parts):
            need = p.cache_needs()
            paged = need.paged if need.paged is not None else paged
            slots += [SlotStateNeed(f"{i}.{s.name}", s.shape, s.dtype) for s in need.slots]
        return CacheNeeds(paged=paged, slots=tuple(slots))

    def scratch_bytes(self, tokens: int) -> int:
        return sum(p.scratch_bytes(tokens) for p in self.parts)          # (the shared matrices are the branches' own, side by side)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        proj = None
        if self.w_all is not None:
            proj = self.ctx.workspace.buffer("parallel.proj", (x.shape[0], self.w_all.shape[0]), self.ctx.dtype)
            ops.scope("parallel.in_projection")
            linear(x, self.w_all, proj, self.b_all)
        pre = None
        if self.w_out is not None:
            pre = self.ctx.workspace.buffer("parallel.pre", (x.shape[0], self.w_out.shape[1]), self.ctx.dtype)
        for i, p in enumerate(self.parts):
            tag = f"{i}."
            own = dataclasses.replace(cache, state={k[len(tag):]: v for k, v in cache.state.items() if k.startswith(tag)})
            if pre is not None:
                (a, b), (c, d) = self.columns[i], self.out_columns[i]
                p.forward_projected(proj[:, a:b], residual, step, own, out=pre[:, c:d])
            elif proj is not None:
                a, b = self.columns[i]
                p.forward_projected(proj[:, a:b], residual, step, own)
            else:
                p.forward(x, residual, step, own)
        if pre is not None:
            ops.scope("parallel.out_projection")
            linear(pre, self.w_out, residual, self.b_out, accumulate=True)


registry.register("mixer", "gated_linear_recurrence", GatedLinearRecurrence)
registry.register("mixer", "decayed_linear_attention", DecayedLinearAttention)
registry.register("mixer", "parallel", ParallelMixers)
