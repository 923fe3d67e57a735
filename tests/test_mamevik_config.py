"""The Mamevik configuration, its mapping to a model description, and the cache manager's caches per run of
a looped layer (no GPU)."""
import copy

import pytest
import torch

import mamevik_cases as cases
from inferloop_b200.cache import CacheManager
from inferloop_b200.config import ConfigError, UnsupportedConfig, read_model_config
from inferloop_b200.config.mamevik import MamevikConfig
from inferloop_b200.models.decoder import DecoderModel, declare_weights
from inferloop_b200.parts.base import BuildContext, SlotStateNeed, Workspace
import json


def spec_of(config):
    return read_model_config(json.dumps(config))[2]


def test_the_run_order_repeats_the_looped_layers_with_a_cache_per_run():
    spec = spec_of(cases.CONFIG_V)
    n = len(cases.CONFIG_V["layers"])
    order = [(e.layer, e.instance) for e in spec.run_order]
    assert order == [(0, 0), (1, 0)] + [x for p in range(3) for x in ((n, p), (2, p), (3, p))]       # the loop reaches the last layer
    assert spec.layers[n].block.kind == "loop_input" and spec.head_name is None and spec.logits_post is None
    u = spec_of(cases.CONFIG_U)
    assert [(e.layer, e.instance) for e in u.run_order][:3] == [(4, 0), (0, 0), (1, 0)]          # the loop starts at the first layer
    assert u.logits_post["cap"] == 10.0 and u.logits_post["scale"] == 2.0
    w = spec_of(cases.CONFIG_W)
    assert len(w.layers) == 4 and w.embedding["buckets"] == 0 and w.embedding.get("keep") is None


def test_the_declared_tensors_and_their_shapes():
    decl = {d.name: tuple(d.shape) for d in declare_weights(spec_of(cases.CONFIG_U))}
    assert decl["embed"] == (211, 72) and decl["bigram"] == (98, 72) and decl["embed.norm"] == (72,)
    assert decl["loop.in"] == (72, 144) and decl["loop.step"] == (2, 72)
    assert decl["l0.mix.in"] == (2 * 48 + 2 * 16 + 4, 72) and decl["l0.mix.conv"] == (48 + 32, 4) and decl["l0.mix.conv.b"] == (80,)
    assert decl["l0.mix.A_log"] == decl["l0.mix.dt_bias"] == decl["l0.mix.D"] == (4,) and decl["l0.mix.norm"] == (48,)
    assert decl["l1.mix.q"] == (24, 72) and decl["l1.mix.dkv"] == (24, 72) and decl["l1.mix.uk"] == (24, 24)
    assert decl["l1.mix.uv"] == (60, 24) and decl["l1.mix.sink"] == (3,) and decl["l1.mix.o"] == (72, 60)
    assert "l1.mlp.router" not in decl and "l1.norm2" in decl            # a layer without feed-forward: its second norm may be stored
    assert decl["l2.mlp.router"] == (3, 72) and decl["l2.mlp.router.b"] == (3,) and decl["l2.mlp.e2.down"] == (72, 16)
    assert "head" not in decl and decl["final.norm"] == (72,)
    assert "bigram" not in {d.name for d in declare_weights(spec_of(cases.CONFIG_W))}


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].update(type="rwkv"), UnsupportedConfig),
    (lambda c: c["layers"][0]["mixer"].update(groups=3), ConfigError),
    (lambda c: c["layers"][0]["mixer"].update(norm_groups=5), ConfigError),
    (lambda c: c["layers"][0]["mixer"].pop("state"), ConfigError),
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=0), ConfigError),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=-4), ConfigError),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), UnsupportedConfig),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), ConfigError),
    (lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0), ConfigError),
    (lambda c: c["loop"].update(stop=9), ConfigError),
    (lambda c: c["loop"].update(start=2), ConfigError),
    (lambda c: c["loop"].update(times=0), ConfigError),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), ConfigError),
    (lambda c: c.update(logit_softcap=-1.0), ConfigError),
    (lambda c: c["norm"].update(eps=0), ConfigError),
    (lambda c: c.pop("width"), ConfigError),
])
def test_refusals(change, error):
    config = copy.deepcopy(cases.CONFIG_U)
    change(config)
    with pytest.raises(error):
        read_model_config(json.dumps(config))


def test_what_is_absent_from_the_file_is_absent_from_the_model():
    config = copy.deepcopy(cases.CONFIG_U)
    for key in ("loop", "embedding", "logit_scale", "logit_softcap"):
        config.pop(key)
    config["layers"][1]["mixer"].pop("mask")
    cfg = MamevikConfig.from_dict(config)
    assert cfg.loop is None and cfg.bigram is None and cfg.logit_scale == 1.0 and cfg.logit_softcap == 0.0
    assert cfg.layers[1].mixer.window is None
    spec = spec_of(config)
    assert spec.logits_post is None and len(spec.run_order) == 4 and all(e.instance == 0 for e in spec.run_order)


def test_every_run_of_a_looped_layer_has_pages_and_state_of_its_own():
    spec = spec_of(cases.CONFIG_V)
    model = DecoderModel(spec, BuildContext(torch.float32, None, Workspace(None)))
    needs = model.cache_needs()
    assert needs[1].slots[0].shape == (8, 128, 64) and needs[1].slots[1].shape == (3, 8 * 64 + 2 * 2 * 128)
    assert needs[2].paged.head_dim == 128 and needs[2].paged.kv_heads == 1 and needs[2].paged.window == 100 and needs[2].paged.value_dim == 0
    assert model.model_slot_needs() == (SlotStateNeed("previous_token", (), torch.int32),)
    m = CacheManager(needs, page_size=16, num_pages=8, max_requests=2, run_order=spec.run_order, model_slots=model.model_slot_needs())
    # layer 0 and the three runs of layer 3 share a group (one latent of 64, window 33); layer 2 has three caches of its own group
    by_need = {(g.need.head_dim, g.need.window): g.layers for g in m.groups}
    assert by_need == {(64, 33): [0, 3, 3, 3], (128, 100): [2, 2, 2]}
    caches = [m.layer_cache(e) for e in spec.run_order]
    assert [c.instance for c in caches] == [0, 0, 0, 0, 0, 1, 1, 1, 2, 2, 2]
    k = [c.k for c in caches]
    assert m.groups[0].layers == [0, 3, 3, 3] and all(x is None for x in k)        # (no device: the ledger alone)
    m.begin("a"); m.ensure("a", 40); m.commit("a", 40)
    assert m.pages_needed("a", 41) == {0: 0, 1: 0}
    m.release("a")
    m.check()
