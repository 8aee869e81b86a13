"""Attention over a cached low-rank latent, without positions (mixer kind `latent_attention`).

    q = W_q h  [heads, d];   c = rms(W_dkv h) * g  [rank];   k_i = Uk_i c,  v_i = Uv_i c  (head i)
    s_ij = scale * q_i . k_j for the keys j a position reads: all earlier ones and itself, or the
    last `window` of them;  p = softmax over those, with exp(sink_i) joining the denominator when
    the layer has a sink;  out = W_o [p v]

Only c is cached (one "kv head" of `rank` elements per token, no values beside it).  The engine
never forms k and v: with q'_i = Uk_i^T q_i the score is q'_i . c_j, and sum_j p_j v_j =
Uv_i (sum_j p_j c_j), so the attention kernels run over the cached latents as keys and as values
with all heads sharing them, between two small per-head products (csrc/latent.cu; a step of up to 16
tokens writes its latents and maps its queries in one launch).  A step is the
same computation however its tokens were cut: a prompt's portion and a single token take the same
path.  W_q and W_dkv are one product.

What a description may add (all spec parameters; absent, the layer is the one above):

  `q_latent` = n    the queries pass a latent of their own: cq = rms(W_dq h) * gq [n], q = W_uq cq
  `rot_dim` = t     positions by rotation: a head's query is [d unrotated | t rotated]; W_dkv gives rank + t
                    rows, the last t (not normed) are ONE rotated key part shared by all heads;
                    s_ij = scale * (qa_i . Uk c_j + qr_i . kr_j).  The cache row is [c | rotated kr]: the score
                    stays one dot product over rank + t elements between [Uk^T qa | rotated qr] and the row,
                    and the kernels' output keeps only its first `rank` columns for Uv.  `position` names the
                    rotation (pairs of neighbours over the first `rotary_dim` of the t elements).
  `own_cache` = False   the layer has no W_dkv: the run order lets it read another layer's rows, written
                    (normed and rotated) by that layer; its own Uk, Uv, queries and everything else.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from . import registry
from .base import CacheNeeds, Mixer, PagedKVNeed
from .linear import linear


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec.get("v_head_dim") or self.d)
        self.rank = int(spec["latent"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        self.has_sink = bool(spec.get("sink", False))
        self.eps = float(spec["eps"])
        self.q_rank = int(spec.get("q_latent") or 0)
        self.tail = int(spec.get("rot_dim") or 0)
        self.own_cache = bool(spec.get("own_cache", True))
        self.position = registry.build("position", spec["position"], ctx) if spec.get("position") is not None else None
        self.rot = int(spec["position"].get("rotary_dim", 0)) if self.position is not None and self.tail else 0
        if self.tail and self.position is not None and not getattr(self.position, "interleaved", False) and self.rot:
            raise ValueError("latent attention: the rotated part turns in pairs of neighbours (position kind rope_interleaved)")
        if self.rot > self.tail:
            raise ValueError(f"latent attention: {self.rot} rotated elements in a part of {self.tail}")
        self.general = bool(self.q_rank or self.tail or not self.own_cache)
        # split-KV decode cuts the keys at multiples of this, fixed per model; with a window the chunks a token reads
        # are few wherever it stands, so they can be short
        self.decode_chunk = ops.DECODE_CHUNK_MIN if self.window else ops.decode_chunk_for(int(spec.get("max_positions", 4096)))
        names = {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "sink": "sink", "o": "o",
                 "q_down": "dq", "q_down_norm": "dq.norm", "q_up": "uq"}
        for role, name in spec.get("names", ()):
            if role not in names:
                raise ValueError(f"latent attention has no tensor role {role!r}")
            names[role] = name
        self.names = {k: prefix + v for k, v in names.items()}
        self.w_in = self.w_o = self.latent_norm = self.up_k = self.up_v = self.sink = self.q_norm = self.w_uq = None

    @property
    def graph_safe(self) -> bool:
        return self.position is None or bool(self.position.graph_safe)

    def declare_weights(self) -> List[WeightDecl]:
        n, H = self.names, self.hidden
        qw = self.heads * (self.d + self.tail)
        if self.q_rank:
            out = [WeightDecl(n["q_down"], (self.q_rank, H)), WeightDecl(n["q_down_norm"], (self.q_rank,), "vector", "norm"),
                   WeightDecl(n["q_up"], (qw, self.q_rank))]
        else:
            out = [WeightDecl(n["q"], (qw, H))]
        if self.own_cache:
            out += [WeightDecl(n["down"], (self.rank + self.tail, H)), WeightDecl(n["down_norm"], (self.rank,), "vector", "norm")]
        out += [WeightDecl(n["up_k"], (self.heads * self.d, self.rank)), WeightDecl(n["up_v"], (self.heads * self.dv, self.rank)),
                WeightDecl(n["o"], (H, self.heads * self.dv))]
        if self.has_sink:
            out.append(WeightDecl(n["sink"], (self.heads,), "vector", "around_zero"))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        first = tensors[n["q_down"]] if self.q_rank else tensors[n["q"]]
        self.w_in = (torch.cat([first, tensors[n["down"]]], dim=0) if self.own_cache else first).contiguous()
        if self.own_cache:
            self.latent_norm = tensors[n["down_norm"]].contiguous()
        if self.q_rank:
            self.q_norm = tensors[n["q_down_norm"]].contiguous()
            self.w_uq = tensors[n["q_up"]].contiguous()
        # [heads, K, N] for out = x W: queries to the latent space (K = d, N = rank), latent sums to values (K = rank, N = dv)
        self.up_k = tensors[n["up_k"]].view(self.heads, self.d, self.rank).contiguous()
        self.up_v = tensors[n["up_v"]].view(self.heads, self.dv, self.rank).transpose(1, 2).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.has_sink:
            self.sink = tensors[n["sink"]].contiguous()

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedKVNeed(1, self.rank + self.tail, self.window, 0))

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        row = self.rank + self.tail
        return tokens * (size * (self.heads * (self.d + self.tail + 2 * row + self.dv) + self.q_rank)
                         + 4 * (self.q_rank + row + self.rot))

    def _forward_general(self, x: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        """The layer with any of: queries through a latent, a rotated part, another layer's cache."""
        T, ws, dt = x.shape[0], self.ctx.workspace, self.ctx.dtype
        H, d, dv, r, tail = self.heads, self.d, self.dv, self.rank, self.tail
        row, qh = r + tail, d + tail
        q_cols = self.q_rank or H * qh
        # a latent that is normed next is kept in 32-bit; queries that are used as they are, in the compute dtype
        proj = ws.buffer("latent.proj", (T, self.w_in.shape[0]), torch.float32 if self.q_rank else dt)
        ops.scope("attention.qkv_projection")
        linear(x, self.w_in, proj)
        if self.q_rank:
            cq = ws.buffer("latent.cq", (T, self.q_rank), dt)
            ops.scope("attention.query_latent_norm")
            ops.group_norm_add(proj[:, :self.q_rank], self.q_norm, self.eps, 1, out=cq)
            q_src = ws.buffer("latent.q_heads", (T, H * qh), dt)
            ops.scope("attention.query_up_projection")
            linear(cq, self.w_uq, q_src)
        else:
            q_src = proj
        table = step.block_tables[cache.group]
        angles = None
        if self.rot:
            ops.scope("attention.position_table")
            angles = self.position.table(step)
        q = ws.buffer("latent.q", (T, H * row), dt)
        write = cache.writable and self.own_cache
        ops.scope("attention.latent_norm_cache_write")
        if write or tail:
            ops.latent_write_rot(proj, q_cols, r, tail, self.rot, angles, self.latent_norm if write else None, self.eps, step,
                                 table if write else None, cache.k if write else None,
                                 q_src if tail else None, q if tail else None, q_col0=d, q_head_stride=qh, heads=H)
        ops.scope("attention.queries_to_latent")
        ops.head_matmul(q_src, self.up_k, q, x_head_stride=qh, out_head_stride=row)
        ops.scope("attention.attention")
        o = ws.buffer("latent.o", (T, H * row), dt)
        ops.attention(q, o, cache.k, cache.k, step, table, self.window or 0, self.scale, H, 1, row, workspace=ws,
                      decode_chunk=self.decode_chunk, sink=self.sink)
        ops.scope("attention.latent_to_values")
        v = ws.buffer("latent.v", (T, H * dv), dt)
        ops.head_matmul(o, self.up_v, v, x_head_stride=row)
        ops.scope("attention.o_projection")
        linear(v, self.w_o, residual, accumulate=True)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        if self.general:
            return self._forward_general(x, residual, step, cache)
        T, ws, dt = x.shape[0], self.ctx.workspace, self.ctx.dtype
        H, d, dv, r = self.heads, self.d, self.dv, self.rank
        proj = ws.buffer("latent.proj", (T, H * d + r), dt)
        ops.scope("attention.qkv_projection")
        linear(x, self.w_in, proj)
        table = step.block_tables[cache.group]
        q = ws.buffer("latent.q", (T, H * r), dt)
        if T <= ops.LATENT_INPUT_TOKENS and cache.writable and cache.k.dtype == dt:
            ops.scope("attention.input_stage (latent norm, cache write, queries to latent)")
            ops.latent_input(proj, self.up_k, q, H * d, r, self.latent_norm, self.eps, step, table, cache.k)
        else:
            ops.scope("attention.latent_norm_cache_write")
            if cache.writable:
                ops.latent_write(proj, H * d, r, self.latent_norm, self.eps, step, table, cache.k)
            ops.scope("attention.queries_to_latent")
            ops.head_matmul(proj, self.up_k, q)
        ops.scope("attention.attention")
        o = ws.buffer("latent.o", (T, H * r), dt)
        ops.attention(q, o, cache.k, cache.k, step, table, self.window or 0, self.scale, H, 1, r, workspace=ws,
                      decode_chunk=self.decode_chunk, sink=self.sink)
        ops.scope("attention.latent_to_values")
        v = ws.buffer("latent.v", (T, H * dv), dt)
        ops.head_matmul(o, self.up_v, v)
        ops.scope("attention.o_projection")
        linear(v, self.w_o, residual, accumulate=True)


registry.register("mixer", "latent_attention", LatentAttention)
