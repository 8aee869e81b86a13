"""The Zebivik configuration, its mapping to a model description, and what its layers ask of the cache manager (no GPU)."""
import copy
import json

import pytest
import torch

import plain_zebivik as plain
import zebivik_cases as cases
from inferloop_b200.cache import CacheManager
from inferloop_b200.config import ConfigError, UnsupportedConfig, read_model_config
from inferloop_b200.config.zebivik import ZebivikConfig
from inferloop_b200.models.decoder import DecoderModel, declare_weights
from inferloop_b200.parts.base import BuildContext, Workspace


def spec_of(config):
    return read_model_config(json.dumps(config))[2]


def test_the_mapping():
    spec = spec_of(cases.CONFIG_K)
    assert spec.architecture == "Zebivik" and spec.head_name == "head" and spec.embedding.kind == "normed"
    assert spec.final_norm.kind == "dyt" and spec.logits_post["cap"] == 6.0
    assert [l.block.kind for l in spec.layers] == ["sandwich"] * 4 and spec.layers[0].block["residual_mult"] == 0.7
    assert [l.mixer.kind for l in spec.layers] == ["parallel", "gated_linear_recurrence", "gated_linear_recurrence", "parallel"]
    assert [l.feed_forward.kind for l in spec.layers] == ["routed_experts", "swiglu", "none", "routed_experts"]
    (lp, left), (rp, right) = spec.layers[0].mixer["branches"]
    assert (lp, rp) == ("left.", "right.") and left.kind == "gqa_attention" and right.kind == "decayed_linear_attention"
    assert left["out_scale"] == 0.9 and right["out_scale"] == 1.3 and left["output_gate"] == "head" and left["bias"] is True
    assert left["position"]["scaling"] == (4.0, 1.0, 3.0, 40.0) and left["position"]["rotary_dim"] == 8
    assert spec.layers[3].mixer["branches"][0][1]["position"].kind == "none"
    ffn = spec.layers[0].feed_forward
    assert ffn["groups"] == (3, 2) and ffn["correction"] and ffn["route_scale"] == 2.0 and ffn["shared_inter"] == 12 and ffn["renorm_eps"] == 1e-20
    assert spec.layers[3].feed_forward["groups"] is None and spec.layers[3].feed_forward["shared_inter"] == 0
    dense = spec.layers[1].feed_forward["activation"]
    assert dense.kind == "clamped_glu" and dense["limit"] == 0.8 and dense["sharpness"] == 1.702 and dense["up_offset"] == 1.0
    assert spec_of(cases.CONFIG_L).logits_post is None


def test_the_declared_tensors_and_their_shapes():
    decl = {d.name: tuple(d.shape) for d in declare_weights(spec_of(cases.CONFIG_K))}
    assert decl["embed"] == (203, 72) and decl["head"] == (203, 72)
    for n in ("embed.norm", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b"):
        assert decl[n] == (72,) and decl[n + ".b"] == (72,) and decl[n + ".alpha"] == ()
    assert decl["l0.mix.left.q"] == (60, 72) and decl["l0.mix.left.k"] == (12, 72) and decl["l0.mix.left.v"] == (10, 72)
    assert decl["l0.mix.left.q.b"] == (60,) and decl["l0.mix.left.o"] == (72, 50) and decl["l0.mix.left.o.b"] == (72,)
    assert decl["l0.mix.left.g"] == (5, 72)
    assert decl["l0.mix.right.q"] == decl["l0.mix.right.k"] == (30, 72) and decl["l0.mix.right.v"] == decl["l0.mix.right.g"] == (18, 72)
    assert decl["l0.mix.right.norm"] == (18,) and decl["l0.mix.right.o"] == (72, 18)
    assert decl["l1.mix.y"] == decl["l1.mix.x"] == (60, 72) and decl["l1.mix.conv"] == (60, 5) and decl["l1.mix.ra"] == (3, 20, 20)
    assert decl["l1.mix.ri.b"] == (3, 20) and decl["l1.mix.lam"] == (60,) and decl["l1.mix.o"] == (72, 60)
    assert decl["l1.mlp.gate"] == (40, 72) and decl["l1.mlp.down"] == (72, 40)
    assert decl["l0.mlp.router"] == (6, 72) and decl["l0.mlp.correction"] == (6,) and decl["l0.mlp.e5.up"] == (20, 72)
    assert decl["l0.mlp.shared.gate"] == (12, 72) and "l3.mlp.shared.gate" not in decl
    assert "l2.mlp.gate" not in decl and "l2.norm2" in decl          # a layer without feed-forward: its norms may be stored
    optional = {d.name for d in declare_weights(spec_of(cases.CONFIG_K)) if d.optional}
    assert {"l2.norm2", "l2.norm2.b", "l2.norm2.alpha", "l2.norm2b"} <= optional and "l1.norm2" not in optional


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].update(type="mamba2"), UnsupportedConfig),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=2), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=14), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].update(high=1.0), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("factor"), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 0.5]), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 0.5, 1.5]), ConfigError),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), ConfigError),
    (lambda c: c["layers"][1]["mixer"].update(blocks=7), ConfigError),
    (lambda c: c["layers"][1]["mixer"].update(conv=17), UnsupportedConfig),
    (lambda c: c["layers"][1]["mlp"].update(limit=0), ConfigError),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), UnsupportedConfig),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), ConfigError),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), ConfigError),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4), ConfigError),
    (lambda c: c.update(logit_softcap=-1.0), ConfigError),
    (lambda c: c["norm"].update(eps=0), ConfigError),
    (lambda c: c.pop("width"), ConfigError),
    (lambda c: c.update(layers=[]), ConfigError),
])
def test_refusals(change, error):
    config = copy.deepcopy(cases.CONFIG_K)
    change(config)
    with pytest.raises(error):
        read_model_config(json.dumps(config))


def test_what_is_absent_from_the_file_is_absent_from_the_model():
    config = copy.deepcopy(cases.CONFIG_K)
    config.pop("logit_softcap"); config.pop("residual_mult")
    config["layers"][0]["mixer"]["left"]["rot"].pop("scaling")
    config["layers"][0]["mlp"]["router"].pop("groups")
    config["layers"][0]["mlp"].pop("shared")
    cfg = ZebivikConfig.from_dict(config)
    assert cfg.logit_softcap == 0.0 and cfg.residual_mult == 1.0 and cfg.layers[0].mixer.left.rot.scaling is None
    assert cfg.layers[0].mlp.groups == 1 and cfg.layers[0].mlp.shared_ff == 0 and cfg.layers[2].mlp is None
    spec = spec_of(config)
    assert spec.logits_post is None and spec.layers[0].mixer["branches"][0][1]["position"]["scaling"] is None


def test_what_the_layers_ask_of_the_cache_manager():
    """A parallel layer: pages for the softmax side, a state slot for the linear side under its branch's number; a
    recurrent layer: its state and the convolution's last inputs; a model of recurrences only has no page group."""
    spec = spec_of(cases.CONFIG_K)
    model = DecoderModel(spec, BuildContext(torch.float32, None, Workspace(None)))
    needs = model.cache_needs()
    assert needs[0].paged.kv_heads == 1 and needs[0].paged.head_dim == 12 and needs[0].paged.value_dim == 10 and needs[0].paged.window is None
    assert [(s.name, s.shape) for s in needs[0].slots] == [("1.state", (3, 10, 6))]
    assert [(s.name, s.shape) for s in needs[1].slots] == [("state", (60,)), ("conv", (4, 60))] and needs[1].paged is None
    assert [(s.name, s.shape) for s in needs[2].slots] == [("state", (24,)), ("conv", (0, 24))]
    m = CacheManager(needs, page_size=4, num_pages=8, max_requests=2, run_order=spec.run_order)
    assert len(m.groups) == 2                      # two softmax geometries, two page groups
    m.begin("a"); m.ensure("a", 9); m.commit("a", 9)
    m.release("a")
    m.check()
    n = DecoderModel(spec_of(cases.CONFIG_N), BuildContext(torch.float32, None, Workspace(None)))
    assert all(x.paged is None for x in n.cache_needs())
    assert len(CacheManager(n.cache_needs(), page_size=16, num_pages=4, max_requests=2).groups) == 0


def test_the_plain_statement_routes_by_groups_and_ranks_with_the_correction():
    """The oracle itself on a case worked by hand: scores that prefer expert 0, a correction that makes the ranking
    prefer the second group, weights from the scores alone."""
    scores = torch.tensor([[0.4, 0.1, 0.3, 0.2]], dtype=torch.float64)
    corr = torch.tensor([0.0, 0.0, 0.15, 0.0], dtype=torch.float64)
    chosen, weights = plain.route(scores, corr, 2, {"count": 2, "keep": 1}, 3.0)
    assert chosen.tolist() == [[2, 3]]                     # group 1 wins with 0.45 against 0.4; inside it 0.45 > 0.2
    assert torch.allclose(weights, torch.tensor([[0.6, 0.4]], dtype=torch.float64) * 3.0)
    chosen, _ = plain.route(scores, corr - 10.0, 1, {"count": 2, "keep": 1}, 1.0)        # every ranking score negative
    assert chosen.tolist() == [[2]]
    chosen, weights = plain.route(scores, corr, 3, None, 1.0)
    assert chosen.tolist() == [[2, 0, 3]] and abs(float(weights.sum()) - 1.0) < 1e-12
