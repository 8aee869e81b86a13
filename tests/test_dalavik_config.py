"""The Dalavik configuration, its mapping to a model description, the declared tensors, and the caches of layers that
read an earlier layer's rows (no GPU)."""
import copy
import json

import pytest
import torch

import dalavik_cases as cases
from inferloop_b200.cache import CacheManager
from inferloop_b200.config import ConfigError, UnsupportedConfig, read_model_config
from inferloop_b200.config.dalavik import DalavikConfig, MixedHeadsMixer, RotatedLatentMixer
from inferloop_b200.models.decoder import DecoderModel, declare_weights
from inferloop_b200.parts.base import BuildContext, Workspace


def spec_of(config):
    return read_model_config(json.dumps(config))[2]


def test_the_file_chooses_the_architecture_and_every_size_comes_from_it():
    arch, cfg, spec = read_model_config(json.dumps(cases.CONFIG_P))
    assert arch.name == "dalavik" and isinstance(cfg, DalavikConfig)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.norm_groups, cfg.side_dim) == (211, 72, 3e-5, 3, 5)
    kinds = [type(l.mixer) for l in cfg.layers]
    assert kinds == [RotatedLatentMixer, MixedHeadsMixer, RotatedLatentMixer, RotatedLatentMixer, MixedHeadsMixer]
    first, reader = cfg.layers[0].mixer, cfg.layers[3].mixer
    assert (first.rot_dim, first.rot_dims, first.rot_base, first.kv_from) == (6, 4, 50.0, None) and reader.kv_from == 0
    assert cfg.layers[1].mlp is None and cfg.layers[0].mlp.ff == 40
    assert cfg.layers[1].mixer.q_temp.every == 3 and cfg.layers[4].mixer.q_temp is None and cfg.layers[4].mixer.softcap == 0.0
    assert spec.architecture == "Dalavik" and spec.head_name is None and spec.embedding_name == "embed"


def test_a_reading_layer_runs_on_the_cache_of_the_layer_it_names():
    spec = spec_of(cases.CONFIG_P)
    assert [(e.layer, e.cache_of, e.writes_cache) for e in spec.run_order] == [
        (0, 0, True), (1, 1, True), (2, 2, True), (3, 0, False), (4, 4, True)]
    model = DecoderModel(spec, BuildContext(torch.float32, None, Workspace(None)))
    needs = model.cache_needs()
    # a latent layer's page rows hold the latent and the rotated part; a reader needs the same rows
    assert needs[0].paged.head_dim == 18 + 6 and needs[0].paged.kv_heads == 1 and needs[2].paged.head_dim == 10 + 4
    assert needs[1].paged.kv_heads == 2 and needs[1].paged.head_dim == 12 and needs[1].paged.value_dim == 20
    m = CacheManager(needs, page_size=4, num_pages=12, max_requests=2, run_order=spec.run_order, model_slots=model.model_slot_needs())
    caches = [m.layer_cache(e) for e in spec.run_order]
    assert caches[3].layer == caches[0].layer and not caches[3].writable and caches[0].writable
    m.begin("a"); m.ensure("a", 9); m.commit("a", 9)
    m.release("a")
    m.begin("b"); m.ensure("b", 30); m.commit("b", 30)
    m.release("b")
    m.check()


def test_the_declared_tensors_and_their_shapes():
    decl = {d.name: tuple(d.shape) for d in declare_weights(spec_of(cases.CONFIG_P))}
    assert decl["embed"] == (211, 72) and decl["side.embed"] == (211, 5 * 5) and decl["final.norm"] == (72,)
    assert decl["l0.mix.dq"] == (20, 72) and decl["l0.mix.dq.norm"] == (20,) and decl["l0.mix.uq"] == (3 * (8 + 6), 20)
    assert decl["l0.mix.dkv"] == (18 + 6, 72) and decl["l0.mix.dkv.norm"] == (18,)
    assert decl["l0.mix.uk"] == (3 * 8, 18) and decl["l0.mix.uv"] == (3 * 10, 18) and decl["l0.mix.o"] == (72, 30)
    assert "l3.mix.dkv" not in decl and "l3.mix.dkv.norm" not in decl and decl["l3.mix.uk"] == (5 * 4, 18)
    assert decl["l1.mix.q"] == (48, 72) and decl["l1.mix.q.b"] == (48,) and decl["l1.mix.k"] == (24, 72) and decl["l1.mix.v.b"] == (40,)
    assert decl["l1.mix.q.norm"] == decl["l1.mix.k.norm"] == (12,) and decl["l1.mix.talk"] == (4, 4)
    assert decl["l1.mix.r1"] == decl["l1.mix.r2"] == decl["l1.mix.sink"] == (4,) and decl["l1.mix.o"] == (72, 80)
    assert "l1.mlp.gate" not in decl and decl["l0.mlp.gate"] == decl["l0.mlp.up"] == (40, 72) and decl["l0.mlp.down"] == (72, 40)
    assert decl["l2.side.gate"] == (5, 72) and decl["l2.side.proj"] == (72, 5) and decl["l2.side.norm"] == (72,)
    assert decl["l0.norm1"] == decl["l0.norm2"] == (72,)
    none = {d.name for d in declare_weights(spec_of(cases.CONFIG_R))}
    assert "side.embed" not in none and "l0.side.gate" not in none


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].update(type="conv"), UnsupportedConfig),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), UnsupportedConfig),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=8), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(base=0.0), ConfigError),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), ConfigError),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), ConfigError),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), ConfigError),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), ConfigError),          # another rank and rotation
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0, kv_rank=18, rot_dim=6, rot={"base": 50.0, "dims": 4}) or
     c["layers"][3]["mixer"].update(kv_from=2), ConfigError),                       # a reader is not read
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), ConfigError),
    (lambda c: c["layers"][1]["mixer"].update(softcap=-1.0), ConfigError),
    (lambda c: c["layers"][1]["mixer"]["q_temp"].pop("every"), ConfigError),
    (lambda c: c["norm"].update(groups=5), ConfigError),
    (lambda c: c["norm"].update(eps=0), ConfigError),
    (lambda c: c.pop("vocab"), ConfigError),
    (lambda c: c.update(layers=[]), ConfigError),
])
def test_refusals(change, error):
    config = copy.deepcopy(cases.CONFIG_P)
    change(config)
    with pytest.raises(error):
        read_model_config(json.dumps(config))


def test_what_is_absent_from_the_file_is_absent_from_the_model():
    cfg = DalavikConfig.from_dict(cases.CONFIG_R)
    assert cfg.side_dim == 0 and cfg.norm_groups == 1
    spec = spec_of(cases.CONFIG_R)
    assert all(l.block.get("extra") is None for l in spec.layers)
    first = spec.layers[0].mixer
    assert first["softcap"] == 0.0 and tuple(first["query_temperature"]) == (1.0, 1)
    assert spec.layers[2].mixer["query_temperature"] is None and spec.layers[2].feed_forward.kind == "none"
