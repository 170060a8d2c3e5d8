"""The Zadinex configuration: what it reads, what it refuses, what it declares (no GPU)."""
import pytest
import torch

from helpers import write_folder
from plain import zadinex_plain as P
from zadinex_cases import CASES, make_config


def test_registered_and_specs_follow_the_description():
    from titan_b200.config import config_from_dict, known_architectures
    assert "Zadinex" in known_architectures()
    cfg = make_config("odd")
    spec = config_from_dict(cfg).to_model_spec()
    assert spec.architecture == "Zadinex" and spec.hidden_size == 56 and spec.vocab_size == 131
    assert [l.mixer.kind for l in spec.layers] == ["wkv", "attention", "attention", "wkv"]
    assert all(l.arrangement == "pre_norm_scaled" and l.mixer_norm.kind == "dyt" for l in spec.layers)
    assert spec.layers[1].feed_forward is None and spec.layers[1].option("scales") == ("ls1",)
    a = spec.layers[1].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.option("value_dim"), a.softmax_scale) == (3, 1, 12, 20, 0.3)
    assert a.position.rotary_dim == 4 and a.position.theta == 500.0 and a.position.pairing == "half"
    assert a.option("unit_norm") == "after_rotation" and a.option("unit_norm_eps") == 3e-6 and a.option("value_mix") is None
    assert spec.layers[2].mixer.option("value_mix") == (None, "vmix")
    f = spec.layers[3].feed_forward
    assert (f.kind, f.activation, f.option("experts"), f.option("identity"), f.option("groups"), f.option("keep"), f.option("limit")) == \
        ("moe", "swish_clamped", 3, 3, 3, 1, 2.5)
    assert spec.layers[0].feed_forward.activation == "gelu_tanh" and spec.layers[0].mixer.option("rank") == 3


def test_later_blending_layers_name_the_first():
    from titan_b200.config import config_from_dict
    spec = config_from_dict(make_config("wide")).to_model_spec()
    assert [l.mixer.option("value_mix") for l in spec.layers] == [None, (None, "vmix"), None, (1, "vmix"), None]


@pytest.mark.parametrize("name", sorted(CASES))
def test_declared_tensors_are_the_plain_list(name):
    from titan_b200.config import config_from_dict
    from titan_b200.parts import declare_weights
    cfg = make_config(name)
    spec = config_from_dict(cfg).to_model_spec()
    declared = {w.name: tuple(w.shape) for w in declare_weights(spec)}
    plain = {n: tuple(s) for n, s, _ in P.tensor_list(cfg)}
    assert all(plain[n] == s for n, s in declared.items())
    assert set(plain) - set(declared) <= set(spec.ignorable_tensors)       # the first blending layer's factor: in the file, used by nobody


def test_rank_comes_from_the_tensor_where_the_description_has_none(tmp_path):
    from titan_b200.config import ConfigError, config_from_dict, load_config
    cfg = make_config("mix")
    weights = {k: v.to(torch.bfloat16) for k, v in P.random_weights(cfg, 1).items()}
    del cfg["layers"][1]["mixer"]["rank"]
    with pytest.raises(ConfigError, match="rank"):
        config_from_dict(cfg)
    write_folder(str(tmp_path), cfg, weights)
    assert load_config(str(tmp_path)).to_model_spec().layers[1].mixer.option("rank") == 5


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0].update(type="conv"), "not known"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "not known"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "experts"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][1]["mlp"]["expert"].update(limit=0.0), "limit"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=24), "blended"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_refusals(change, match):
    from titan_b200.config import ConfigError, config_from_dict
    cfg = make_config("mix")
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(cfg)


def test_parts_refuse_what_they_cannot_run():
    from titan_b200.config import FeedForwardSpec, MixerSpec
    from titan_b200.parts import FEED_FORWARDS, MIXERS
    with pytest.raises(ValueError):
        FEED_FORWARDS.build(FeedForwardSpec("moe", 32, 16, "swish_clamped", extra=(("experts", 4), ("top", 2))))      # no limit
    with pytest.raises(ValueError):
        FEED_FORWARDS.build(FeedForwardSpec("moe", 32, 16, "silu", extra=(("experts", 4), ("top", 2), ("identity", 2))))      # pass-through experts need the other routing
    with pytest.raises(ValueError):
        FEED_FORWARDS.build(FeedForwardSpec("moe", 32, 16, "silu", extra=(("experts", 6), ("top", 3), ("routing", "softmax_all"), ("groups", 3), ("keep", 1))))
    with pytest.raises(ValueError):
        MIXERS.build(MixerSpec("wkv", 32, 2, head_dim=300, extra=(("rank", 4),)))
    with pytest.raises(ValueError):
        MIXERS.build(MixerSpec("attention", 32, 2, 2, 16, extra=(("unit_norm", "sideways"),)))


def test_the_plain_router_keeps_to_open_groups_and_counts_negative_scores():
    """The oracle itself: with every corrected score negative, an expert of a closed group (whose score would be 'zero' if
    closed groups were zeroed instead of removed) must not be chosen."""
    f = {"router": {"experts": 4, "top": 2, "identity": 2, "groups": {"count": 3, "keep": 1}}}
    h = torch.eye(6, dtype=torch.float64)[:3]
    W = {"r.router": torch.randn(6, 6, generator=torch.Generator().manual_seed(3)).double(),
         "r.correction": torch.full((6,), -5.0, dtype=torch.float64)}
    idx, w = P.routed_choice(h, f, W, "r.")
    assert all(int(a) // 2 == int(b) // 2 for a, b in idx.tolist())         # both from one group
    assert torch.allclose(w.sum(-1), torch.ones(3, dtype=torch.float64))


def test_a_folder_of_random_weights_is_written_and_read_back(tmp_path):
    """The random-weights mode on this design: tensors without dimensions (a norm's factor, a blending factor) included."""
    from titan_b200.config import config_from_dict, load_config
    from titan_b200.parts import declare_weights
    from titan_b200.weights import FolderWeights, write_model_folder
    folder = write_model_folder(str(tmp_path / "m"), config_from_dict(make_config("odd")), seed=4)
    cfg = load_config(folder)
    declared = declare_weights(cfg.to_model_spec())
    source = FolderWeights(folder, declared, torch.float32, "cpu")
    by_name = {w.name: w for w in declared}
    assert "l2.mix.vmix" not in by_name                      # the only blending layer: nobody uses its factor, so it is not written
    assert source.get(by_name["l0.norm1.alpha"]).shape == () and source.get(by_name["final.norm.alpha"]).dtype == torch.float32
    assert source.get(by_name["l0.mix.w2"]).shape == (40, 3)


def test_factors_of_switched_off_mechanisms_may_be_in_the_file(tmp_path):
    """A layer that does not blend values may still carry its factor, a layer without feed-forward its second norm and scale."""
    from titan_b200.config import load_config
    from titan_b200.parts import declare_weights
    from titan_b200.weights import FolderWeights, WeightError
    cfg = make_config("odd")
    weights = {k: v.to(torch.bfloat16) for k, v in P.random_weights(cfg, 2).items()}
    weights["l1.mix.vmix"] = torch.tensor(0.5, dtype=torch.bfloat16)
    weights["l1.ls2"] = torch.ones(cfg["width"], dtype=torch.bfloat16)
    folder = write_folder(str(tmp_path / "m"), cfg, weights)
    spec = load_config(folder).to_model_spec()
    assert "l1.mix.vmix" in spec.ignorable_tensors and "l1.ls2" in spec.ignorable_tensors and "l0.ls2" not in spec.ignorable_tensors
    FolderWeights(folder, declare_weights(spec), torch.float32, "cpu", spec.ignorable_tensors)
    with pytest.raises(WeightError):
        FolderWeights(folder, declare_weights(spec), torch.float32, "cpu")
