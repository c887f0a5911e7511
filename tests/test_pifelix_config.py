"""The Pifelix configuration, its tensors, its caches and the cache manager's handling of chunked masks, without a GPU."""
import copy

import pytest

from pifelix_helpers import CONFIG_A, CONFIG_B, CONFIG_C


def _spec(d):
    from transformers_neuronx_b200.config import config_from_dict
    arch, cfg = config_from_dict(copy.deepcopy(d))
    return arch, cfg, arch.build_spec(cfg)


def test_the_architecture_is_found_by_its_single_name_and_round_trips():
    from transformers_neuronx_b200.config import PifelixConfig, config_from_dict
    arch, cfg, spec = _spec(CONFIG_A)
    assert arch.name == "Pifelix" and isinstance(cfg, PifelixConfig)
    again = config_from_dict(cfg.to_dict())[1]
    assert again == cfg and again.to_dict()["layers"] == CONFIG_A["layers"]
    assert spec.vocab_size == 211 and spec.hidden_size == 72 and len(spec.layers) == 4
    assert spec.embedding.scale == 3.7 and all(l.residual_scale == 0.45 and l.block == "output_norm" for l in spec.layers)


def test_tensor_names_and_shapes_follow_the_layers():
    from transformers_neuronx_b200.models.decoder import DecoderModel
    _, _, spec = _spec(CONFIG_A)
    t = {s.name: tuple(s.shape) for s in DecoderModel(spec).tensor_specs()}
    assert t["embed"] == (211, 72) and t["head"] == (211, 72) and t["final.norm"] == (72,)
    assert t["l0.mix.q"] == (144, 72) and t["l0.mix.q.b"] == (144,) and t["l0.mix.k"] == (48, 72) and t["l0.mix.v"] == (80, 72)
    assert t["l0.mix.q.conv"] == (144, 4) and t["l0.mix.k.conv"] == (48, 4) and t["l0.mix.v.conv"] == (80, 4)
    assert t["l0.mix.q.norm"] == (24,) and t["l0.mix.k.norm"] == (24,)          # one weight vector for all heads
    assert t["l0.mix.o"] == (72, 240) and "l0.mix.o.b" not in t
    assert t["l0.mlp.router"] == (5, 72) and t["l0.mlp.e4.gate"] == (36, 72) and t["l0.mlp.e4.down"] == (72, 36)
    assert "l0.mlp.e5.gate" not in t and "l0.mlp.e0.gate.b" not in t
    # a layer that reads another layer's keys and values has none of their tensors; this one has no feed-forward either
    assert t["l1.mix.q"] == (144, 72) and t["l1.mix.q.conv"] == (144, 4) and t["l1.mix.q.norm"] == (24,)
    for gone in ("l1.mix.k", "l1.mix.v", "l1.mix.k.b", "l1.mix.k.conv", "l1.mix.v.conv", "l1.mix.k.norm", "l1.norm2", "l1.mlp.router"):
        assert gone not in t
    _, _, spec_b = _spec(CONFIG_B)
    tb = {s.name: tuple(s.shape) for s in DecoderModel(spec_b).tensor_specs()}
    assert "l1.mix.q.conv" not in tb and tb["l3.mix.q.conv"] == (96, 1)          # no convolution; a single tap


def test_pages_state_and_what_a_reading_layer_keeps():
    from transformers_neuronx_b200.cache import FixedStateNeed, PagedKVNeed, group_needs
    from transformers_neuronx_b200.models.decoder import DecoderModel
    _, _, spec = _spec(CONFIG_A)
    needs = DecoderModel(spec).cache_needs()
    assert needs[(0, 0)] == PagedKVNeed(2, 48, None, 20)               # keys of 24 and values of 40 in pages of 48
    assert needs[(0, 1)] == FixedStateNeed((3, 144 + 48 + 80), "activation")
    assert needs[(1, 0)] == FixedStateNeed((3, 144), "activation") and (1, 1) not in needs      # its queries' past only
    assert needs[(2, 0)] == PagedKVNeed(1, 64, None, None)             # read under another mask too: nothing given back early
    assert needs[(3, 0)] == FixedStateNeed((1, 128), "activation")
    groups = [g for g in group_needs(needs) if g.paged]
    assert [(g.chunk, g.cache_ids) for g in groups] == [(20, [(0, 0)]), (None, [(2, 0)])]
    _, _, spec_b = _spec(CONFIG_B)
    nb = DecoderModel(spec_b).cache_needs()
    assert nb[(1, 0)] == PagedKVNeed(4, 64, None, None) and (1, 1) not in nb     # no convolution: no state
    assert nb[(3, 0)] == PagedKVNeed(1, 96, None, 48) and (3, 1) not in nb       # one tap keeps nothing either


def test_pages_before_the_running_chunk_go_back_to_the_pool():
    from transformers_neuronx_b200.cache import CacheManager, PagedKVNeed, group_needs
    cm = CacheManager(group_needs({0: PagedKVNeed(1, 16, None, 40)}), page_size=16, num_pages=6, max_slots=2)
    cm.add_request("a")
    cm.append("a", 39)                                   # positions 0..38: chunk 0 still runs
    assert cm.release_behind_window("a") == 0 and cm.free_pages() == [3]
    cm.append("a", 1)                                    # position 39 is the chunk's last; the next query opens chunk 1
    assert cm.release_behind_window("a") == 2            # blocks 0 and 1 (positions 0..31); block 2 holds 40..47 as well
    assert cm.block_table("a")[:3] == [-1, -1, cm.block_table("a")[2]] and cm.block_table("a")[2] >= 0
    cm.append("a", 41)                                   # positions 40..80: chunk 2 begins at 80
    assert cm.release_behind_window("a") == 3 and cm.free_pages() == [5]
    cm.check()
    with pytest.raises(ValueError, match="behind the window"):
        cm.slot_of_position("a", 50)
    cm.free_request("a")
    assert cm.free_pages() == [6]


@pytest.mark.parametrize("edit, word", [
    (lambda d: d["layers"][0].update(type="mamba"), "unknown layer type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=4), "cannot share"),
    (lambda d: d["layers"][2]["mixer"].update(rot={"dims": 66, "base": 9.0}), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"].update(scale=0.0), "scale must be positive"),
    (lambda d: d["layers"][0]["mixer"].update(kv_from=0), "earlier layer"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=1), "no keys and values of its own"),
    (lambda d: d["layers"][1]["mixer"].update(vdim=24), "vdim differs"),
    (lambda d: d["layers"][1]["mixer"].update(rot={"dims": 16, "base": 7.0}), "rotation differs"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind must be 'moe'"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=6), "exceeds"),
    (lambda d: d["layers"][0]["mixer"].update(mask={"size": 0}), "size"),
    (lambda d: d.pop("residual_mult"), "residual_mult"),
    (lambda d: d["embedding"].pop("scale"), "scale"),
])
def test_a_configuration_that_cannot_be_run_is_refused_by_name(edit, word):
    from transformers_neuronx_b200.config import ConfigError, config_from_dict
    d = copy.deepcopy(CONFIG_A)
    edit(d)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_stretched_frequencies_follow_the_ramp():
    """Against numbers worked out by hand: 8 dims, base 100, original context 40, fast 4, slow 1, factor 5."""
    import math
    from transformers_neuronx_b200.parts.rotary import inverse_frequencies, rotation_magnitude
    from transformers_neuronx_b200.parts.spec import FrequencyRampSpec
    s = FrequencyRampSpec(5.0, 40.0, 4.0, 1.0)
    turns = lambda t: 8 * math.log(40 / (2 * math.pi * t)) / (2 * math.log(100))
    lo, hi = max(math.floor(turns(4.0)), 0), min(math.ceil(turns(1.0)), 7)
    assert (lo, hi) == (0, 2)
    f = inverse_frequencies(8, 100.0, "cpu", s).double()
    plain = [100 ** (-2 * i / 8) for i in range(4)]
    want = [plain[0], plain[1] * (0.5 / 5 + 0.5), plain[2] / 5, plain[3] / 5]
    assert all(abs(float(f[i]) - want[i]) <= 1e-7 * want[i] for i in range(4))
    assert abs(rotation_magnitude(s) - (0.1 * math.log(5.0) + 1)) < 1e-12 and rotation_magnitude(None) == 1.0
    assert float((inverse_frequencies(8, 100.0, "cpu").double() - __import__("torch").tensor(plain)).abs().max()) < 1e-7


def test_all_configurations_build():
    for d in (CONFIG_A, CONFIG_B, CONFIG_C):
        _, _, spec = _spec(d)
        assert len(spec.schedule) == len(d["layers"])
