"""Grouped-query causal attention over the paged cache, with optional per-head q/k
RMSNorm, optional biases, optional window, and a position encoding chosen by spec.

Order of operations as in the reference's decoder recipe
(crates/model/recipes/src/decoder.rs:229-364): q/k/v projections; per-head RMSNorm of q
and k over head_dim with a weight [head_dim] shared by all heads (:278-293), before the
rotation (:315-335); cache append (:336-342); attention with head h reading kv head
h / (nq / nkv) and scale 1/sqrt(head_dim)
(crates/testing/cpu/reference-ops/src/kernels.rs:251-297); output projection added to the
residual (:358-363).  Biases, where the spec asks for them, are added in 32-bit right
after each projection.

The three projection matrices are concatenated at load into one [(nq + nkv) d + nkv dv, H]
matrix so one GEMM produces q|k|v.

What a description may vary beyond that (all spec parameters, the defaults give the layer
above): `v_head_dim` (values of another head size than queries and keys), `bias` = True /
False / "qkv" (no bias on the output projection), `qk_norm` = True (weight [head_dim]) or
"unweighted" (q and k divided by their root mean square), `qk_norm_after_rotation`,
`scale` (the multiplier of q.k), a position kind whose pairs are interleaved, tensor names
(`names`: pairs (role, name under the prefix)), and `value_mix` = "first" | "mixed": the first
such layer of a model keeps its values of the step's tokens, every later one caches
(1 - lambda) v + lambda v_first with its own learned scalar lambda.

Scores may be reshaped and mixed across heads before the softmax (each a spec parameter, absent by
default; any of them sends the layer to the kernel that owns a token with all its heads,
csrc/attention_mix.cu): `query_temperature` = (coef, every): q at position i is multiplied by
1 + coef ln(floor((i + 1) / every) + 1); `softcap` = c: s <- c tanh(s / c); `distance_bias`: s <- s -
r1_h ln(1 + r2_h (i - j)) with two learned vectors; `head_mix`: s_h <- sum_g M[h, g] s_g with a learned
[heads, heads] matrix; in that order.  `sink`: a learned logit per head joins the softmax's denominator.

`output_gate` = "head": head h's output is multiplied by sigmoid((W_g x)_h), one number a head from a matrix
[heads, hidden] whose rows ride behind q|k|v in the one projection.  `out_scale`: a constant on the whole mixer's
output (a mixer that runs beside another one), applied in 32-bit to what the output projection reads and to its bias.
"""
from __future__ import annotations

import math
from typing import List, Mapping, Optional

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from . import registry
from .base import CacheNeeds, Mixer, PagedKVNeed
from .linear import linear


class GQAttention(Mixer):
    @property
    def graph_safe(self) -> bool:
        """The kernels read the batch from device memory; the position encoding answers for itself."""
        return bool(self.position.graph_safe)

    def __init__(self, spec, ctx, prefix: str = "") -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.nq = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads are not a multiple of {self.nkv} kv heads")
        self.dv = int(spec.get("v_head_dim") or self.d)
        qk_norm = spec.get("qk_norm", False)
        if qk_norm not in (False, True, "unweighted"):
            raise ValueError(f"qk_norm must be False, True or 'unweighted', found {qk_norm!r}")
        self.qk_norm = qk_norm is True                       # with a weight per head element
        self.qk_norm_unweighted = qk_norm == "unweighted"
        self.qk_norm_after = bool(spec.get("qk_norm_after_rotation", False))
        self.qk_norm_eps = float(spec.get("qk_norm_eps", 1e-6))
        bias = spec.get("bias", False)
        if bias not in (False, True, "qkv"):
            raise ValueError(f"bias must be False, True or 'qkv', found {bias!r}")
        self.bias = bool(bias)                               # q, k, v
        self.out_bias = bias is True
        self.window = spec.get("window")
        self.scale = float(spec["scale"]) if spec.get("scale") is not None else 1.0 / math.sqrt(self.d)
        self.value_mix = spec.get("value_mix")
        if self.value_mix not in (None, "first", "mixed"):
            raise ValueError(f"value_mix must be None, 'first' or 'mixed', found {self.value_mix!r}")
        # split-KV decode cuts the keys at multiples of this, fixed per model so that the
        # cut never depends on the batch
        self.decode_chunk = ops.decode_chunk_for(int(spec.get("max_positions", 4096)))
        temp = spec.get("query_temperature")
        self.temp_coef, self.temp_every = (float(temp[0]), int(temp[1])) if temp else (0.0, 1)
        if temp and self.temp_every <= 0:
            raise ValueError("query_temperature: the period must be positive")
        self.softcap = float(spec.get("softcap") or 0.0)
        self.distance_bias = bool(spec.get("distance_bias", False))
        self.head_mix = bool(spec.get("head_mix", False))
        self.has_sink = bool(spec.get("sink", False))
        self.output_gate = spec.get("output_gate")
        if self.output_gate not in (None, "head"):
            raise ValueError(f"output_gate must be None or 'head', found {self.output_gate!r}")
        self.out_scale = float(spec.get("out_scale", 1.0))
        if self.out_scale != 1.0 and not self.output_gate:
            raise ValueError("attention: a constant on the output is applied by the gate's kernel (output_gate)")
        self.gate_rows = -(-self.nq // 8) * 8 if self.output_gate else 0      # (padded: the projection's rows stay multiples of 16 bytes)
        self.shaped = bool(self.temp_coef or self.softcap or self.distance_bias or self.head_mix)
        if self.shaped and self.value_mix is not None:
            raise ValueError("attention: reshaped scores and mixed values are not served together")
        self.position = registry.build("position", spec["position"], ctx)
        self.rotary_dim = int(spec["position"].get("rotary_dim", 0))
        p = prefix
        names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                 "qb": "q_proj.bias", "kb": "k_proj.bias", "vb": "v_proj.bias", "ob": "o_proj.bias",
                 "qn": "q_norm.weight", "kn": "k_norm.weight", "vmix": "v_mix",
                 "r1": "r1", "r2": "r2", "head_mix": "talk", "sink": "sink", "g": "gate.weight"}
        for role, name in spec.get("names", ()):
            if role not in names:
                raise ValueError(f"attention has no tensor role {role!r}")
            names[role] = name
        self.names = {k: p + v for k, v in names.items()}
        self.mode = ((ops.ROPE_INTERLEAVED if getattr(self.position, "interleaved", False) else 0)
                     | (ops.NORM_AFTER_ROTATION if self.qk_norm_after else 0)
                     | (ops.NORM_UNWEIGHTED if self.qk_norm_unweighted else 0))
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_norm = self.k_norm = self.v_lambda = None
        self.r1 = self.r2 = self.mix = self.sink = None

    # ------------------------------------------------------------------ weights
    def declare_weights(self) -> List[WeightDecl]:
        n, d, dv, H = self.names, self.d, self.dv, self.hidden
        out = [WeightDecl(n["q"], (self.nq * d, H)), WeightDecl(n["k"], (self.nkv * d, H)),
               WeightDecl(n["v"], (self.nkv * dv, H)), WeightDecl(n["o"], (H, self.nq * dv))]
        if self.bias:
            out += [WeightDecl(n["qb"], (self.nq * d,), "vector", "bias"),
                    WeightDecl(n["kb"], (self.nkv * d,), "vector", "bias"),
                    WeightDecl(n["vb"], (self.nkv * dv,), "vector", "bias")]
        if self.out_bias:
            out.append(WeightDecl(n["ob"], (H,), "vector", "bias"))
        if self.qk_norm:
            out += [WeightDecl(n["qn"], (d,), "vector", "norm"),
                    WeightDecl(n["kn"], (d,), "vector", "norm")]
        if self.distance_bias:
            out += [WeightDecl(n["r1"], (self.nq,), "vector", "positive"), WeightDecl(n["r2"], (self.nq,), "vector", "positive")]
        if self.head_mix:
            out.append(WeightDecl(n["head_mix"], (self.nq, self.nq), "vector", "eye"))
        if self.has_sink:
            out.append(WeightDecl(n["sink"], (self.nq,), "vector", "around_zero"))
        if self.output_gate:
            out.append(WeightDecl(n["g"], (self.nq, H)))
        if self.value_mix == "mixed":
            out.append(WeightDecl(n["vmix"], (), "vector", "mix"))
        elif bool(self.spec.get("value_mix_tensor_unused", False)):
            out.append(WeightDecl(n["vmix"], (), "vector", "mix", optional=True))    # stored, never read
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        rows = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]]
        if self.output_gate:
            g = tensors[n["g"]]
            rows += [g, g.new_zeros(self.gate_rows - self.nq, self.hidden)]
        self.w_qkv = torch.cat(rows, dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.bias:
            biases = [tensors[n["qb"]], tensors[n["kb"]], tensors[n["vb"]]]
            if self.output_gate:
                biases.append(biases[0].new_zeros(self.gate_rows))
            self.b_qkv = torch.cat(biases).contiguous()
        if self.out_bias:
            self.b_o = (tensors[n["ob"]] * self.out_scale).contiguous() if self.out_scale != 1.0 else tensors[n["ob"]].contiguous()
        if self.value_mix == "mixed":
            self.v_lambda = tensors[n["vmix"]].reshape(1).contiguous()
        if self.qk_norm:
            self.q_norm = tensors[n["qn"]].contiguous()
            self.k_norm = tensors[n["kn"]].contiguous()
        if self.distance_bias:
            self.r1, self.r2 = tensors[n["r1"]].contiguous(), tensors[n["r2"]].contiguous()
        if self.head_mix:
            self.mix = tensors[n["head_mix"]].contiguous()
        if self.has_sink:
            self.sink = tensors[n["sink"]].contiguous()

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedKVNeed(self.nkv, self.d, self.window, self.dv if self.dv != self.d else None))

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        width = (self.nq + self.nkv) * self.d + self.nkv * self.dv + self.gate_rows
        kept = self.nkv * self.dv if self.value_mix else 0
        return tokens * ((width + self.nq * (self.d + self.dv) + kept) * size + self.rotary_dim * 4)

    # ------------------------------------------------------------------ run
    def input_rows(self):
        """(matrix, bias or None) of the one product this mixer starts with: a mixer that runs beside others can have its
        rows stacked with theirs (see `forward_projected`).  The matrix may be replaced by a view of the stacked one."""
        return self.w_qkv, self.b_qkv

    def take_input_rows(self, rows: torch.Tensor) -> None:
        """The same matrix as a view of the stacked one: no second copy is kept."""
        self.w_qkv = rows

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        T = x.shape[0]
        ws, dt = self.ctx.workspace, self.ctx.dtype
        width = (self.nq + self.nkv) * self.d + self.nkv * self.dv + self.gate_rows
        qkv = ws.buffer("attn.qkv", (T, width), dt)
        ops.scope("attention.qkv_projection")
        linear(x, self.w_qkv, qkv, self.b_qkv)
        self.forward_projected(qkv, residual, step, cache)

    def output_rows(self):
        """(matrix [hidden, heads * v_head_dim], bias or None) of the product this mixer ends with, or None when its input
        cannot be written elsewhere (no gate kernel in between): a mixer that runs beside others can have its columns
        stacked with theirs (`forward_projected(..., out=...)`)."""
        return (self.w_o, self.b_o) if self.output_gate else None

    def forward_projected(self, qkv: torch.Tensor, residual: torch.Tensor, step, cache, out: Optional[torch.Tensor] = None) -> None:
        """The mixer from its projection's output on: `qkv` [T, q | k | v (| gates)], rows of any stride.  With `out`
        [T, heads * v_head_dim] (rows of any stride) the gated attention output goes there and the output product is left to
        the caller."""
        T = qkv.shape[0]
        ws, dt = self.ctx.workspace, self.ctx.dtype
        gate_col0 = (self.nq + self.nkv) * self.d + self.nkv * self.dv      # the heads' gate logits ride behind q | k | v
        table = step.block_tables[cache.group]
        ops.scope("attention.position_table")
        rope = self.position.table(step)
        v_first = None
        if self.value_mix is not None:
            # the step's tokens' values of the first layer that mixes: kept by it, read by the later ones
            v_first = ws.buffer(f"attn.v_first/{self.nkv}x{self.dv}", (T, self.nkv * self.dv), dt)
        if (self.dv == self.d and step.decode_only and cache.k is not None and (cache.writable or self.value_mix is None)
                and not self.shaped and not self.has_sink
                and ops.attention_decode_fused_supported(
                    dt, cache.k.dtype, self.nq, self.nkv, self.d, cache.page_size, self.rotary_dim, rope is not None,
                    interleaved=bool(self.mode & ops.ROPE_INTERLEAVED))):
            # one token per sequence: norm, rotation and the cache write of the new key and
            # value happen inside the attention kernel
            o = ws.buffer("attn.o", (T, self.nq * self.d), dt)
            ops.scope("attention.decode (q/k norm, rotation, cache write inside)")
            ops.attention_decode_fused(qkv, o, self.q_norm, self.k_norm, self.qk_norm_eps, rope, cache.k, cache.v,
                                       cache.writable, step.positions, step.cu_q, table, self.window or 0, self.scale,
                                       step.n_seqs, self.nq, self.nkv, self.d,
                                       long_context=step.max_kv_len >= ops.DECODE_LONG_CONTEXT, mode=self.mode,
                                       rotary_dim=self.rotary_dim or None, v_first=v_first,
                                       v_lambda=self.v_lambda if self.value_mix == "mixed" else None,
                                       v_keep=self.value_mix == "first")
            self._finish(o, qkv, gate_col0, residual, out)
            return
        q = ws.buffer("attn.q", (T, self.nq * self.d), dt)
        ops.scope("attention.qk_norm_rotation_cache_write")
        ops.qk_norm_rope_cache(
            qkv, q, self.q_norm, self.k_norm, self.qk_norm_eps, rope,
            self.rotary_dim, step.positions, step.seq_of_token, table, cache.page_size,
            cache.k if cache.writable else None, cache.v if cache.writable else None,
            self.nq, self.nkv, self.d, self.dv, self.mode, v_first=v_first,
            v_lambda=self.v_lambda if self.value_mix == "mixed" else None, v_keep=self.value_mix == "first")
        o = ws.buffer("attn.o", (T, self.nq * self.dv), dt)
        ops.scope("attention.attention")
        if self.shaped:
            ops.attention_mixed_heads(q, o, cache.k, cache.v, step, table, self.window or 0, self.scale, self.nq, self.nkv,
                                      self.d, self.dv, sink=self.sink, head_mix=self.mix, dist_r1=self.r1, dist_r2=self.r2,
                                      softcap=self.softcap, temp_coef=self.temp_coef, temp_every=self.temp_every,
                                      workspace=ws, decode_chunk=ops.DECODE_CHUNK_MIN)
        else:
            ops.attention(q, o, cache.k, cache.v, step, table, self.window or 0, self.scale,
                          self.nq, self.nkv, self.d, workspace=ws, decode_chunk=self.decode_chunk, dv=self.dv, sink=self.sink)
        self._finish(o, qkv, gate_col0, residual, out)

    def _finish(self, o: torch.Tensor, qkv: torch.Tensor, gate_col0: int, residual: torch.Tensor, out: Optional[torch.Tensor]) -> None:
        """The gate a head and the mixer's constant on what the output product reads, then that product (or, with `out`,
        the gated rows into the caller's matrix)."""
        if self.output_gate:
            ops.scope("attention.output_gate")
            ops.head_gate(o, qkv[:, gate_col0:], self.nq, self.out_scale, out=out)
        elif out is not None:
            raise ops.KernelError("attention: without a gate the output product is the mixer's own")
        if out is None:
            ops.scope("attention.o_projection")
            linear(o, self.w_o, residual, self.b_o, accumulate=True)


registry.register("mixer", "gqa_attention", GQAttention)
