"""The Tefezen configuration on the CPU: keys read, refusals, the parts it asks for, the tensors it declares."""
import copy

import pytest
import torch

from plain import tefezen_plain as P
from tefezen_cases import CASES, make_config

from titan_b200.config import ConfigError, TefezenConfig, config_from_dict
from titan_b200.parts import declare_weights


@pytest.mark.parametrize("name", sorted(CASES))
def test_declared_tensors_are_the_designs(name):
    cfg = make_config(name)
    spec = config_from_dict(cfg).to_model_spec()
    declared = {w.name: tuple(w.shape) for w in declare_weights(spec)}
    assert declared == {n: tuple(s) for n, s, _ in P.tensor_list(cfg)}
    assert len(spec.layers) == len(cfg["layers"]) and spec.order == tuple(range(len(cfg["layers"])))
    assert all(layer.arrangement == "output_norm" for layer in spec.layers)


def test_the_name_may_stand_alone_or_in_a_list():
    cfg = make_config("small")
    assert isinstance(config_from_dict(cfg), TefezenConfig)
    cfg2 = dict(cfg)
    cfg2["architectures"] = [cfg2.pop("architecture")]
    assert isinstance(config_from_dict(cfg2), TefezenConfig)
    with pytest.raises(ConfigError, match="not registered"):
        config_from_dict(dict(cfg, architecture="Nothing"))


def test_constants_come_from_the_file():
    cfg = make_config("odd")
    spec = config_from_dict(cfg).to_model_spec()
    assert spec.embedding_scale == cfg["embedding"]["scale"]
    for layer, lc in zip(spec.layers, cfg["layers"]):
        m = lc["mixer"]
        assert layer.mixer_norm.eps == cfg["norm"]["eps"] and layer.mixer_norm.weight_offset == 1.0
        if lc["type"] == "latent_attention":
            assert layer.mixer.window == m["mask"]["size"] and layer.mixer.softmax_scale == m["scale"]
            assert layer.mixer.position.theta == m["rot"]["base"] and layer.mixer.position.rotary_dim == m["rot"]["dims"]
            assert layer.mixer.position.pairing == "adjacent" and layer.mixer.cache_from == m.get("kv_from")
            assert layer.mixer.option("latent_norm").weight_offset == 0.0
        else:
            assert layer.mixer.option("decay") == tuple(m["decay"])
        if lc.get("mlp"):
            f = layer.feed_forward
            assert (f.option("experts"), f.option("top")) == (lc["mlp"]["router"]["experts"], lc["mlp"]["router"]["top"])
            assert f.option("shared_size") == (lc["mlp"].get("shared") or {}).get("ff", 0)
        else:
            assert layer.feed_forward is None and layer.feed_forward_norm is None
        side = layer.option("sublayers")
        assert len(side) == 1 and side[0].option("offset") == layer.index * cfg["token_side"]["dim"]
    # without the keys: no scale, no token input, no shared expert
    bare = make_config("bare")
    spec = config_from_dict(bare).to_model_spec()
    assert spec.embedding_scale is None and spec.shared_tensors == () and spec.layers[0].option("sublayers") == ()


def test_an_owner_keeps_what_its_longest_reader_sees():
    cfg = make_config("odd")          # layer 3 reads layer 0's rows with a longer window than layer 0's own
    spec = config_from_dict(cfg).to_model_spec()
    readers = [l for l in spec.layers if l.mixer.cache_from is not None]
    assert readers
    for l in readers:
        owner = spec.layers[l.mixer.cache_from]
        assert owner.mixer.option("cache_window") >= max(l.mixer.window, owner.mixer.window)
    from titan_b200.parts import MIXERS
    need = MIXERS.build(spec.layers[0].mixer).cache_need()
    assert need.kind == "latent" and need.window == spec.layers[0].mixer.option("cache_window")
    assert need.head_dim % 8 == 0 and need.head_dim >= cfg["layers"][0]["mixer"]["kv_rank"] + cfg["layers"][0]["mixer"]["rot_dim"]
    assert MIXERS.build(readers[0].mixer).cache_need() is None


@pytest.mark.parametrize("edit,message", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0].update(type="convolution"), "not known"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=99), "experts"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not known"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "keeps no latents"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=5), "earlier layer"),
    (lambda c: c.update(layers=[]), "at least one layer"),
])
def test_refusals_name_the_key(edit, message):
    cfg = copy.deepcopy(make_config("small"))
    edit(cfg)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(cfg)


def test_a_reader_must_share_the_rows_meaning():
    cfg = copy.deepcopy(make_config("small"))
    cfg["layers"][2]["mixer"]["kv_rank"] += 8
    with pytest.raises(ConfigError, match="kv_rank"):
        config_from_dict(cfg).to_model_spec()
    cfg = copy.deepcopy(make_config("small"))
    cfg["layers"][2]["mixer"]["rot"]["base"] *= 2
    with pytest.raises(ConfigError, match="rotates"):
        config_from_dict(cfg).to_model_spec()


def test_a_latent_group_keeps_one_plane_and_a_ring():
    from titan_b200.cache import CacheNeed, SequenceCache
    cache = SequenceCache([CacheNeed("latent", 1, 40, 70), CacheNeed("state", state_shape=(2, 4, 8)), None],
                          max_tokens=640, max_slots=3, max_context=640, dtype=torch.float32, device="cpu")
    latent, state = cache.groups
    assert latent.storage.shape == (1, 1, 10, 1, 64, 40) and latent.ring_rows == 128 and latent.table_width == 2
    s = cache.alloc_slot()
    cache.reserve({s: 500})
    assert len(latent.pages_of[s]) == 2                 # a ring never holds more than its pages
    state.storage[0, s] = 7.0
    cache.free_slot(s)
    assert cache.alloc_slot() == s and float(state.storage[0, s].abs().sum()) == 0.0        # a state starts from zero again
    cache.check()
