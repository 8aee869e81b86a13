"""Residual blocks.

Pre-norm (`pre_norm`): h += mixer(norm1(h)); h += ffn(norm2(h))
(crates/model/recipes/src/decoder.rs:112-120 and :474-480).

Norm on the sublayer's output (`output_norm`): h += norm1(mixer(h)); h += norm2(ffn(h)); and, when the
layer has one, a third sublayer fed by the token itself: h += norm3(extra(h, token)).  The sublayers read
the stream as it is (in the compute dtype); each adds into a zeroed 32-bit buffer, and one kernel norms
that buffer, adds it to the stream, hands the next sublayer its input and zeroes the buffer again.

Norms on both sides (`sandwich`): h += m * norm1b(mixer(norm1(h))); h += m * norm2b(ffn(norm2(h))) with a constant
multiplier m on what joins the stream.  The norms are element-wise (Dynamic Tanh), so the norm on a sublayer's
output, the sum into the stream and the norm in front of the next sublayer are one launch."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..csrc import ops
from ..weights.decl import WeightDecl
from . import registry
from .base import Block, CacheNeeds
from .norm import DynamicTanh, RMSNorm


class PreNormBlock(Block):
    """spec: hidden_size, and the tensor-name pieces of this arrangement:
    mixer_prefix, ffn_prefix, mixer_norm, ffn_norm (names under the layer prefix)."""

    def __init__(self, spec, ctx, prefix: str = "", layer=None) -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        mixer_prefix = prefix + spec.get("mixer_prefix", "self_attn.")
        ffn_prefix = prefix + spec.get("ffn_prefix", "mlp.")
        norm_cls_args = dict(width=self.hidden)
        self.norm1 = registry.build_norm(layer.norm, ctx, prefix + spec.get("mixer_norm", "input_layernorm."), **norm_cls_args)
        self.norm2 = registry.build_norm(layer.norm, ctx, prefix + spec.get("ffn_norm", "post_attention_layernorm."), **norm_cls_args)
        self.mixer = registry.build("mixer", layer.mixer, ctx, mixer_prefix)
        self.ffn = registry.build("feed_forward", layer.feed_forward, ctx, ffn_prefix)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in (self.norm1, self.mixer, self.norm2, self.ffn))

    def declare_weights(self) -> List[WeightDecl]:
        second = self.norm2.declare_weights()
        if getattr(self.ffn, "absent", False):        # the absent sublayer's norm may be stored; it is not read
            second = [WeightDecl(d.name, d.shape, d.role, d.init, d.root, True) for d in second]
        return self.norm1.declare_weights() + self.mixer.declare_weights() + second + self.ffn.declare_weights()

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        absent = getattr(self.ffn, "absent", False)
        for part in (self.norm1, self.mixer) + (() if absent else (self.norm2, self.ffn)):
            part.bind(tensors)

    def cache_needs(self) -> CacheNeeds:
        return self.mixer.cache_needs()

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        return tokens * self.hidden * size + self.mixer.scratch_bytes(tokens) + self.ffn.scratch_bytes(tokens)

    def forward(self, hidden: torch.Tensor, step, cache) -> None:
        ws = self.ctx.workspace
        normed = ws.buffer("block.normed", hidden.shape, self.ctx.dtype)
        ops.scope("norm")
        self.norm1.forward(hidden, normed)
        ops.scope("mixer")
        self.mixer.forward(normed, hidden, step, cache)
        if getattr(self.ffn, "absent", False):        # a layer that has only its mixer
            return
        ops.scope("norm")
        self.norm2.forward(hidden, normed)
        ops.scope("feed_forward")
        self.ffn.forward(normed, hidden, step)


class OutputNormBlock(Block):
    """spec: hidden_size; tensor-name pieces mixer_prefix, ffn_prefix, mixer_norm, ffn_norm (under the layer prefix);
    optionally `extra` (a PartSpec of role feed_forward: the third sublayer), `extra_prefix`, `extra_norm` (the
    PartSpec of its norm; default: the layer's) and `extra_norm_name`."""

    def __init__(self, spec, ctx, prefix: str = "", layer=None) -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.norm1 = registry.build_norm(layer.norm, ctx, prefix + spec.get("mixer_norm", "norm1"), width=self.hidden)
        self.norm2 = registry.build_norm(layer.norm, ctx, prefix + spec.get("ffn_norm", "norm2"), width=self.hidden)
        self.mixer = registry.build("mixer", layer.mixer, ctx, prefix + spec.get("mixer_prefix", "mix."))
        self.ffn = registry.build("feed_forward", layer.feed_forward, ctx, prefix + spec.get("ffn_prefix", "mlp."))
        self.has_ffn = not getattr(self.ffn, "absent", False)
        self.extra = self.norm3 = None
        if spec.get("extra") is not None:
            self.extra = registry.build("feed_forward", spec["extra"], ctx, prefix + spec.get("extra_prefix", "side."))
            self.norm3 = registry.build_norm(spec.get("extra_norm") or layer.norm, ctx,
                                             prefix + spec.get("extra_norm_name", "side.norm"), width=self.hidden)
        for n in (self.norm1, self.norm2, self.norm3):
            if n is not None and not isinstance(n, RMSNorm):
                raise ValueError("output_norm: the norms of a sublayer's output must be RMS norms (plain or in groups)")

    PREPARED = "output_norm.prepared"       # memo key: (stream, copy, buffer, shape) that the block before left ready

    def _sublayers(self):
        """(norm, run(x, y, step, cache)) in order."""
        out = [(self.norm1, lambda x, y, step, cache: self.mixer.forward(x, y, step, cache))]
        if self.has_ffn:
            out.append((self.norm2, lambda x, y, step, cache: self.ffn.forward(x, y, step)))
        if self.extra is not None:
            out.append((self.norm3, lambda x, y, step, cache: self.extra.forward(x, y, step)))
        return out

    @property
    def graph_safe(self) -> bool:
        parts = [self.norm1, self.mixer] + ([self.norm2, self.ffn] if self.has_ffn else []) \
            + ([self.norm3, self.extra] if self.extra is not None else [])
        return all(p.graph_safe for p in parts)

    def declare_weights(self) -> List[WeightDecl]:
        out = self.norm1.declare_weights() + self.mixer.declare_weights()
        second = self.norm2.declare_weights()
        if not self.has_ffn:          # the absent sublayer's norm may be stored; it is not read
            second = [WeightDecl(d.name, d.shape, d.role, d.init, d.root, True) for d in second]
        out += second + self.ffn.declare_weights()
        if self.extra is not None:
            out += self.extra.declare_weights() + self.norm3.declare_weights()
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        parts = [self.norm1, self.mixer] + ([self.norm2, self.ffn] if self.has_ffn else []) \
            + ([self.extra, self.norm3] if self.extra is not None else [])
        for part in parts:
            part.bind(tensors)

    def cache_needs(self) -> CacheNeeds:
        return self.mixer.cache_needs()

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        subs = [self.mixer.scratch_bytes(tokens), self.ffn.scratch_bytes(tokens) if self.has_ffn else 0,
                self.extra.scratch_bytes(tokens) if self.extra is not None else 0]
        return tokens * self.hidden * (size + 4) + max(subs)

    def forward(self, hidden: torch.Tensor, step, cache) -> None:
        ws = self.ctx.workspace
        x = ws.buffer("block.normed", hidden.shape, self.ctx.dtype)          # what a sublayer reads
        y = ws.buffer("block.sublayer_out", hidden.shape, torch.float32)     # what it adds into
        subs = self._sublayers()
        # The last norm of a block also leaves the stream's copy and the zeroed buffer for the block that runs
        # next; the step's memo says so (the decoder forgets it before a block of another kind).
        memo = getattr(step, "memo", None)
        prepared = (hidden.data_ptr(), x.data_ptr(), y.data_ptr(), tuple(hidden.shape))
        if memo is None or memo.pop(self.PREPARED, None) != prepared:
            ops.scope("norm")
            ops.cast_zero(hidden, x, y)
        for i, (norm, run) in enumerate(subs):
            ops.scope("mixer" if i == 0 else "feed_forward")
            run(x, y, step, cache)
            ops.scope("norm")
            if i + 1 < len(subs) or memo is not None:
                ops.group_norm_add(y, norm.weight, norm.eps, norm.groups, x=hidden, out=x, zero=True)
            else:
                ops.group_norm_add(y, norm.weight, norm.eps, norm.groups, x=hidden)
        if memo is not None:
            memo[self.PREPARED] = prepared


class SandwichBlock(Block):
    """spec: hidden_size; residual_mult (default 1); tensor-name pieces mixer_prefix, ffn_prefix, mixer_norm, mixer_out_norm,
    ffn_norm, ffn_out_norm (under the layer prefix).  The layer's norm must be of kind `dyt`."""

    # memo key: what the block before left ready: (the zeroed 32-bit buffer, the stream's shape, the block whose input
    # the compute-dtype buffer already holds or None)
    PREPARED = "sandwich.prepared"

    def __init__(self, spec, ctx, prefix: str = "", layer=None) -> None:
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.mult = float(spec.get("residual_mult", 1.0))
        make = lambda key, default: registry.build_norm(layer.norm, ctx, prefix + spec.get(key, default), width=self.hidden)
        self.norm1, self.norm1b = make("mixer_norm", "norm1"), make("mixer_out_norm", "norm1b")
        self.norm2, self.norm2b = make("ffn_norm", "norm2"), make("ffn_out_norm", "norm2b")
        self.mixer = registry.build("mixer", layer.mixer, ctx, prefix + spec.get("mixer_prefix", "mix."))
        self.ffn = registry.build("feed_forward", layer.feed_forward, ctx, prefix + spec.get("ffn_prefix", "mlp."))
        self.has_ffn = not getattr(self.ffn, "absent", False)
        for n in (self.norm1, self.norm1b, self.norm2, self.norm2b):
            if not isinstance(n, DynamicTanh):
                raise ValueError("sandwich: the norms around a sublayer must be element-wise (kind 'dyt')")

        self.successor = None

    def hand_over_to(self, block) -> None:
        """`block` always runs right after this one: this block's last launch norms the new stream for it too."""
        if isinstance(block, SandwichBlock) and block.hidden == self.hidden:
            self.successor = block

    @property
    def graph_safe(self) -> bool:
        return bool(self.mixer.graph_safe and (not self.has_ffn or self.ffn.graph_safe))

    def declare_weights(self) -> List[WeightDecl]:
        second = self.norm2.declare_weights() + self.norm2b.declare_weights()
        if not self.has_ffn:          # the absent sublayer's norms may be stored; they are not read
            second = [WeightDecl(d.name, d.shape, d.role, d.init, d.root, True) for d in second]
        return (self.norm1.declare_weights() + self.norm1b.declare_weights() + self.mixer.declare_weights() + second
                + self.ffn.declare_weights())

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in (self.norm1, self.norm1b, self.mixer) + ((self.norm2, self.norm2b, self.ffn) if self.has_ffn else ()):
            part.bind(tensors)

    def cache_needs(self) -> CacheNeeds:
        return self.mixer.cache_needs()

    def scratch_bytes(self, tokens: int) -> int:
        size = torch.empty((), dtype=self.ctx.dtype).element_size()
        return tokens * self.hidden * (size + 4) + max(self.mixer.scratch_bytes(tokens), self.ffn.scratch_bytes(tokens) if self.has_ffn else 0)

    def forward(self, hidden: torch.Tensor, step, cache) -> None:
        ws = self.ctx.workspace
        x = ws.buffer("block.normed", hidden.shape, self.ctx.dtype)          # what a sublayer reads
        y = ws.buffer("block.sublayer_out", hidden.shape, torch.float32)     # what it adds into
        memo = getattr(step, "memo", None)
        left = memo.pop(self.PREPARED, None) if memo is not None else None
        ops.scope("norm")
        if left is None or left[:2] != (y.data_ptr(), tuple(hidden.shape)):
            ops.cast_zero(hidden, x, y)
            left = None
        if left is None or left[2] != id(self):
            self.norm1.forward(hidden, x)
        ops.scope("mixer")
        self.mixer.forward(x, y, step, cache)
        ops.scope("norm")
        nxt = self.successor if memo is not None else None
        handed = dict(next_norm=nxt.norm1.tensors, out=x) if nxt is not None else {}
        if self.has_ffn:
            ops.dyt_add(y, self.norm1b.tensors, self.mult, hidden, next_norm=self.norm2.tensors, out=x, zero=True)
            ops.scope("feed_forward")
            self.ffn.forward(x, y, step)
            ops.scope("norm")
            ops.dyt_add(y, self.norm2b.tensors, self.mult, hidden, zero=True, **handed)
        else:
            ops.dyt_add(y, self.norm1b.tensors, self.mult, hidden, zero=True, **handed)
        if memo is not None:
            memo[self.PREPARED] = (y.data_ptr(), tuple(hidden.shape), id(nxt) if nxt is not None else None)


registry.register("block", "pre_norm", PreNormBlock)
registry.register("block", "sandwich", SandwichBlock)
registry.register("block", "output_norm", OutputNormBlock)
