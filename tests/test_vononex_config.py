"""The Vononex configuration, its tensors and its caches, without a GPU."""
import copy

import pytest

from vononex_helpers import CONFIG_P, CONFIG_Q


def _spec(d):
    from transformers_neuronx_b200.config import config_from_dict
    arch, cfg = config_from_dict(copy.deepcopy(d))
    return arch, cfg, arch.build_spec(cfg)


def test_the_architecture_is_found_by_its_single_name_and_round_trips():
    from transformers_neuronx_b200.config import VononexConfig, config_from_dict
    arch, cfg, spec = _spec(CONFIG_P)
    assert arch.name == "Vononex" and isinstance(cfg, VononexConfig)
    again = config_from_dict(cfg.to_dict())[1]
    assert again == cfg and again.to_dict()["layers"] == CONFIG_P["layers"]
    assert spec.vocab_size == 211 and spec.hidden_size == 72 and len(spec.layers) == 4


def test_tensor_names_and_shapes_follow_the_layers():
    from transformers_neuronx_b200.models.decoder import DecoderModel
    _, _, spec = _spec(CONFIG_P)
    t = {s.name: tuple(s.shape) for s in DecoderModel(spec).tensor_specs()}
    assert t["embed"] == (211, 72) and t["head"] == (211, 72) and t["final.norm"] == (72,)
    assert t["l0.mix.z"] == (40, 72) and t["l0.mix.z.b"] == (40,) and t["l0.mix.o"] == (72, 40) and "l0.mix.g.b" not in t
    assert "l0.norm2" not in t and "l0.mlp.gate" not in t            # the first layer has no feed-forward
    assert t["l1.mix.left.q"] == (6 * 24, 72) and t["l1.mix.left.k"] == (2 * 24, 72) and t["l1.mix.left.v"] == (2 * 40, 72)
    assert t["l1.mix.left.q.norm"] == (144,) and t["l1.mix.left.k.norm"] == (48,) and t["l1.mix.left.temp"] == (6,)
    assert t["l1.mix.left.o"] == (72, 240) and t["l1.mix.left.o.b"] == (72,)
    assert t["l1.mix.right.q"] == (60, 72) and t["l1.mix.right.v"] == (72, 72) and t["l1.mix.right.g"] == (72, 72)
    assert t["l1.mix.right.o"] == (72, 72) and "l1.mix.right.q.b" not in t and "l1.mix.right.o.b" not in t
    assert t["l2.mlp.gate"] == (50, 72) and t["l2.mlp.down"] == (72, 50) and t["l2.mlp.down.b"] == (72,)


def test_a_parallel_layer_keeps_pages_and_a_state_and_a_recurrent_layer_a_state():
    from transformers_neuronx_b200.cache import FixedStateNeed, PagedKVNeed, group_needs
    from transformers_neuronx_b200.models.decoder import DecoderModel
    _, _, spec = _spec(CONFIG_P)
    needs = DecoderModel(spec).cache_needs()
    assert needs[0] == FixedStateNeed((40,), "float32")
    assert needs[(1, 0)] == PagedKVNeed(2, 48, None)                  # keys of 24 and values of 40 in pages of 48
    assert needs[(1, 1)] == FixedStateNeed((3, 24, 20), "float32")
    assert needs[(2, 0)] == PagedKVNeed(1, 64, None) and needs[3] == FixedStateNeed((33,), "float32")
    groups = group_needs(needs)
    assert sorted(g.key[0] for g in groups) == ["paged", "state"]
    assert [g for g in groups if g.paged][0].cache_ids == [(1, 0), (2, 0)]


@pytest.mark.parametrize("edit, word", [
    (lambda d: d["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda d: d["layers"][1]["mixer"]["right"].update(decay=[0.9]), "one number per head"),
    (lambda d: d["layers"][1]["mixer"]["left"].update(kv_heads=4), "cannot share"),
    (lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=26), "rot.dims"),
    (lambda d: d["layers"][2]["mlp"].update(kind="experts"), "kind must be 'dense'"),
    (lambda d: d.pop("postln_alpha"), "postln_alpha"),
    (lambda d: d["norm"].pop("eps"), "eps"),
])
def test_a_configuration_that_cannot_be_run_is_refused_by_name(edit, word):
    from transformers_neuronx_b200.config import ConfigError, config_from_dict
    d = copy.deepcopy(CONFIG_P)
    edit(d)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_both_configurations_build():
    for d in (CONFIG_P, CONFIG_Q):
        _, _, spec = _spec(d)
        assert len(spec.schedule) == len(d["layers"])
