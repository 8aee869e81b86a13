"""Zebivik decoder: from its typed config to a :class:`ModelSpec`.

The embedding is the token's row, normed.  Every norm is a Dynamic Tanh (tanh(alpha x) g + b, no statistics).  A
layer norms both what a sublayer reads and what it gives, and adds the result times a constant (block kind
`sandwich`).  A mixer is either two mixers side by side on the same input (`parallel`): grouped-query softmax
attention with biases, a partial half-split rotation whose frequencies are rescaled by wavelength, values of their
own head size and a sigmoid gate per head, beside a linear attention with a constant decay per head whose heads are
RMS-normed together and gated, each side times its own constant; or a gated linear recurrence behind a short
convolution (`gated_linear_recurrence`).  The feed-forward is a clamped gated unit, or routed experts (softmax
scores, a correction that only ranks, groups of which the best stay, weights renormalised and scaled) with a
shared expert, or absent.  The output matrix is a tensor of its own; logits are soft-capped.

Tensor names: `embed`, `embed.norm`, `final.norm`, `head` (a norm `n` has `n`, `n.b`, `n.alpha`), and under `l<i>.`:
`norm1`, `norm1b`, `norm2`, `norm2b`, `mix.left.{q,k,v,o}` (+ `.b`), `mix.left.g`, `mix.right.{q,k,v,g,o,norm}`, or
`mix.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o}`; `mlp.{gate,up,down}` or `mlp.router`, `mlp.correction`,
`mlp.e<j>.{gate,up,down}`, `mlp.shared.{gate,up,down}`.
"""
from __future__ import annotations

from ..config.registry import Architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec
from ..config.zebivik import DenseFeedForward, ParallelMixer, ZebivikConfig

# The design fixes these: the dense unit's gate a(g) = g * sigmoid(1.702 g) and the one added to its clamped linear
# half; the rate of the recurrence's decay, log a = -8 r softplus(lam); what joins the sum the chosen scores are
# divided by.
GATE_SHARPNESS = 1.702
UP_OFFSET = 1.0
DECAY_RATE = 8.0
RENORM_EPS = 1e-20

GLU_NAMES = (("gate", "gate"), ("up", "up"), ("down", "down"))


def build_spec(cfg: ZebivikConfig) -> ModelSpec:
    norm = PartSpec.make("dyt", weight_suffix="")
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, ParallelMixer):
            a, b = m.left, m.right
            position = PartSpec.make("none")
            if a.rot is not None:
                s = a.rot.scaling
                position = PartSpec.make("rope_neox", theta=a.rot.base, rotary_dim=a.rot.dims,
                                         scaling=None if s is None else (s.factor, s.low, s.high, s.original))
            left = PartSpec.make(
                "gqa_attention", hidden_size=cfg.width, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim,
                v_head_dim=a.vdim, bias=True, scale=a.scale, max_positions=cfg.max_positions, position=position,
                output_gate="head", out_scale=m.left_scale,
                names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("qb", "q.b"), ("kb", "k.b"), ("vb", "v.b"), ("ob", "o.b"),
                       ("g", "g")))
            right = PartSpec.make(
                "decayed_linear_attention", hidden_size=cfg.width, heads=b.heads, head_dim=b.dim, v_head_dim=b.vdim,
                decay=b.decay, eps=cfg.eps, out_scale=m.right_scale)
            mixer = PartSpec.make("parallel", branches=(("left.", left), ("right.", right)))
        else:
            mixer = PartSpec.make("gated_linear_recurrence", hidden_size=cfg.width, width=m.width, blocks=m.blocks, taps=m.conv,
                                  rate=DECAY_RATE)
        f = layer.mlp
        if f is None:
            ffn = PartSpec.make("none")
        elif isinstance(f, DenseFeedForward):
            ffn = PartSpec.make("swiglu", hidden_size=cfg.width, intermediate_size=f.ff, names=GLU_NAMES,
                                activation=PartSpec.make("clamped_glu", limit=f.limit, sharpness=GATE_SHARPNESS, up_offset=UP_OFFSET))
        else:
            ffn = PartSpec.make(
                "routed_experts", hidden_size=cfg.width, experts=f.experts, top_k=f.top, expert_inter=f.ff, score="softmax",
                renormalize=True, renorm_eps=RENORM_EPS, route_scale=f.scale, weight_on="output", correction=True,
                groups=(f.groups, f.keep) if f.groups > 1 else None, shared_inter=f.shared_ff, shared_gate=False,
                shared_names=GLU_NAMES,
                names=(("router", "router"), ("correction", "correction"), ("gate", "e{e}.gate"), ("up", "e{e}.up"),
                       ("down", "e{e}.down"), ("shared_prefix", "shared.")))
        block = PartSpec.make("sandwich", hidden_size=cfg.width, residual_mult=cfg.residual_mult, mixer_prefix="mix.",
                              ffn_prefix="mlp.", mixer_norm="norm1", mixer_out_norm="norm1b", ffn_norm="norm2", ffn_out_norm="norm2b")
        layers.append(LayerSpec(prefix=f"l{i}.", block=block, mixer=mixer, feed_forward=ffn, norm=norm))
    post = PartSpec.make("soft_cap", cap=cfg.logit_softcap, scale=1.0) if cfg.logit_softcap > 0 else None
    return ModelSpec(
        architecture="Zebivik",
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        embedding_name="embed",
        head_name="head",
        final_norm_name="final.norm",
        final_norm=norm,
        layers=tuple(layers),
        weight_prefixes=("",),
        logits_post=post,
        embedding=PartSpec.make("normed", hidden_size=cfg.width, norm=norm, norm_name="embed.norm"),
    )


ARCHITECTURE = Architecture(
    name="zebivik",
    claims=("Zebivik", "zebivik"),
    read_config=ZebivikConfig.from_dict,
    build_spec=build_spec,
)
