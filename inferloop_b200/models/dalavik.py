"""Dalavik decoder: from its typed config to a :class:`ModelSpec`.

A layer norms what its sublayers GIVE, not what they read (block kind `output_norm`):
x <- x + n1(mixer(x)); x <- x + n2(ff(x)); x <- x + n3(side(x, token)).  The model's norm divides each of
`groups` equal parts of a row by that part's root mean square; the side input's norm is a plain RMS norm.
Mixers: attention over a cached latent with the queries through a latent of their own and a rotated part
shared by all heads (`latent_attention` with `q_latent`, `rot_dim`; a layer may read an earlier layer's
cache), or grouped-query attention with biases, a per-head norm of q and k, a query temperature, capped
scores, a distance term, scores mixed across heads and a sink (`gqa_attention` with those parameters).
The feed-forward is a gated unit with relu; the side input gates a slice of a second token table.  The
output matrix is the token table.

Tensor names: `embed`, `side.embed`, `final.norm`, and under `l<i>.`: `norm1`, `norm2`,
`mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o}` or `mix.{q,q.b,k,k.b,v,v.b,q.norm,k.norm,r1,r2,talk,sink,o}`,
`mlp.{gate,up,down}`, `side.{gate,proj,norm}`.
"""
from __future__ import annotations

from ..config.dalavik import DalavikConfig, RotatedLatentMixer
from ..config.registry import Architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def build_spec(cfg: DalavikConfig) -> ModelSpec:
    norm = PartSpec.make("rms", eps=cfg.eps, weight_suffix="", groups=cfg.norm_groups)
    n = len(cfg.layers)
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, RotatedLatentMixer):
            mixer = PartSpec.make(
                "latent_attention", hidden_size=cfg.width, heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim, latent=m.kv_rank,
                scale=m.scale, eps=cfg.eps, max_positions=cfg.max_positions, q_latent=m.q_rank, rot_dim=m.rot_dim,
                own_cache=m.kv_from is None,
                position=PartSpec.make("rope_interleaved", theta=m.rot_base, rotary_dim=m.rot_dims) if m.rot_dims else None)
            order.append(RunEntry(i, i) if m.kv_from is None else RunEntry(i, m.kv_from, writes_cache=False))
        else:
            mixer = PartSpec.make(
                "gqa_attention", hidden_size=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                v_head_dim=m.vdim, bias="qkv", qk_norm=True, qk_norm_eps=cfg.eps, scale=m.scale,
                max_positions=cfg.max_positions, position=PartSpec.make("none"),
                query_temperature=None if m.q_temp is None else (m.q_temp.coef, m.q_temp.every), softcap=m.softcap,
                distance_bias=True, head_mix=True, sink=True,
                names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("qb", "q.b"), ("kb", "k.b"), ("vb", "v.b"),
                       ("qn", "q.norm"), ("kn", "k.norm"), ("r1", "r1"), ("r2", "r2"), ("head_mix", "talk"), ("sink", "sink")))
            order.append(RunEntry(i, i))
        f = layer.mlp
        if f is None:
            ffn = PartSpec.make("none")
        else:
            ffn = PartSpec.make("swiglu", hidden_size=cfg.width, intermediate_size=f.ff, activation="relu",
                                names=(("gate", "gate"), ("up", "up"), ("down", "down")))
        extra = None
        if cfg.side_dim:
            extra = PartSpec.make("token_gated", hidden_size=cfg.width, dim=cfg.side_dim, column=i * cfg.side_dim,
                                  vocab_size=cfg.vocab, table_width=n * cfg.side_dim, table="side.embed")
        block = PartSpec.make("output_norm", hidden_size=cfg.width, mixer_prefix="mix.", ffn_prefix="mlp.", mixer_norm="norm1",
                              ffn_norm="norm2", extra=extra, extra_prefix="side.", extra_norm_name="side.norm",
                              extra_norm=PartSpec.make("rms", eps=cfg.eps, weight_suffix=""))
        layers.append(LayerSpec(prefix=f"l{i}.", block=block, mixer=mixer, feed_forward=ffn, norm=norm))
    return ModelSpec(
        architecture="Dalavik",
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        embedding_name="embed",
        head_name=None,
        final_norm_name="final.norm",
        final_norm=norm,
        layers=tuple(layers),
        run_order=tuple(order),
        weight_prefixes=("",),
    )


ARCHITECTURE = Architecture(
    name="dalavik",
    claims=("Dalavik", "dalavik"),
    read_config=DalavikConfig.from_dict,
    build_spec=build_spec,
)
