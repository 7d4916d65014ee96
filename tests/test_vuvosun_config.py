"""The Vuvosun configuration: what it reads, what it refuses, what it declares; the cache with several needs a layer; the plain
implementation's own mechanisms against cases worked by hand (no GPU)."""
import numpy as np
import pytest
import torch

from helpers import write_folder
from plain import vuvosun_plain as P
from vuvosun_cases import CASES, make_config, random_weights, tensor_shapes


def test_registered_and_specs_follow_the_description():
    from titan_b200.config import config_from_dict, known_architectures
    assert "Vuvosun" in known_architectures()
    spec = config_from_dict(make_config("odd")).to_model_spec()
    assert (spec.architecture, spec.hidden_size, spec.vocab_size, spec.streams, spec.lm_head) == ("Vuvosun", 56, 131, 3, None)
    assert spec.embedding_norm.weight == "embed.norm" and spec.embedding_norm.eps == 3e-6
    assert [l.mixer.kind for l in spec.layers] == ["mlstm", "parallel", "parallel", "mlstm"]
    assert all(l.arrangement == "hyper" and l.option("streams") == 3 and l.mixer_norm.kind == "rmsnorm" for l in spec.layers)
    assert spec.layers[1].feed_forward is None and spec.layers[1].option("connections") == ("hc1",)
    assert spec.layers[2].option("connections") == ("hc1", "hc2")
    a, r = spec.layers[1].mixer.option("branches")
    assert (a.kind, a.num_heads, a.num_kv_heads, a.head_dim, a.option("value_dim"), a.softmax_scale, a.window) == ("attention", 3, 1, 12, 20, 0.3, 7)
    assert (a.position.rotary_dim, a.position.theta, a.position.pairing) == (4, 500.0, "adjacent")
    assert (a.option("keep_first"), a.option("value_norm"), a.option("sink"), a.option("out_gate"), a.option("output_scale")) == (0, 3e-6, "sink", "g", 1.5)
    assert (r.kind, r.num_heads, r.num_kv_heads, r.head_dim, r.option("value_dim"), r.option("taps"), r.option("output_scale")) == ("gated_delta", 2, 2, 20, 8, 2, 0.5)
    assert spec.layers[2].mixer.option("branches")[0].option("keep_first") == 2
    m = spec.layers[3].mixer
    assert (m.num_heads, m.head_dim, m.option("value_dim"), m.option("gate_cap")) == (2, 20, 24, 6.0)
    f = spec.layers[0].feed_forward
    assert (f.kind, f.activation, f.intermediate_size, f.option("act_eps")) == ("mlp", "polynorm", 33, 3e-6)


def test_an_attention_without_a_mask_sees_every_key():
    from titan_b200.config import config_from_dict
    spec = config_from_dict(make_config("wide")).to_model_spec()
    a = spec.layers[1].mixer.option("branches")[0]
    assert a.window is None and a.option("keep_first") == 0
    assert spec.streams == 1


@pytest.mark.parametrize("name", sorted(CASES))
def test_declared_tensors_are_the_list_written_by_hand(name):
    from titan_b200.config import config_from_dict
    from titan_b200.parts import declare_weights
    cfg = make_config(name)
    declared = {w.name: tuple(w.shape) for w in declare_weights(config_from_dict(cfg).to_model_spec())}
    assert declared == tensor_shapes(cfg)


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(keep_first=-1), "count"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].pop("size"), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(conv=0), "conv"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0.0), "gate_cap"),
    (lambda c: c["layers"][0].update(type="conv"), "not known"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "not known"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c.update(streams=9), "streams"),
    (lambda c: c.pop("streams"), "streams"),
    (lambda c: c.pop("width"), "width"),
])
def test_refusals(change, match):
    from titan_b200.config import ConfigError, config_from_dict
    cfg = make_config("mix")
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(cfg)


def test_parts_refuse_what_they_cannot_run():
    from titan_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, NormSpec
    from titan_b200.parts import FEED_FORWARDS, MIXERS, build_block
    with pytest.raises(ValueError):
        MIXERS.build(MixerSpec("gated_delta", 32, 3, 2, 8))                                     # heads no multiple of key heads
    with pytest.raises(ValueError):
        MIXERS.build(MixerSpec("gated_delta", 32, 2, 2, 300))                                   # more key dimensions than the kernel holds
    with pytest.raises(ValueError):
        MIXERS.build(MixerSpec("mlstm", 32, 2, head_dim=8))                                     # no cap
    with pytest.raises(ValueError):
        MIXERS.build(MixerSpec("parallel", 32))                                                 # no branches
    with pytest.raises(ValueError):
        MIXERS.build(MixerSpec("parallel", 32, extra=(("branches", (MixerSpec("mlstm", 48, 2, head_dim=8, extra=(("gate_cap", 5.0),)),)),)))
    with pytest.raises(ValueError):
        FEED_FORWARDS.build(FeedForwardSpec("mlp", 32, 16, "silu"))
    mixer = MixerSpec("mlstm", 32, 2, head_dim=8, extra=(("gate_cap", 5.0),))
    with pytest.raises(ValueError):
        build_block(LayerSpec(0, "hyper", mixer, None, NormSpec("rmsnorm", 32, 1e-5, "n"), None, "l0.", extra=(("connections", ("hc1",)),)))      # no streams
    with pytest.raises(ValueError):
        build_block(LayerSpec(0, "hyper", mixer, None, NormSpec("rmsnorm", 32, 1e-5, "n"), None, "l0.", extra=(("connections", ("hc1", "hc2")), ("streams", 2))))


def test_several_streams_need_the_arrangement_that_keeps_them():
    from titan_b200.config import ConfigError, config_from_dict
    import dataclasses
    spec = config_from_dict(make_config("mix")).to_model_spec()
    plain = dataclasses.replace(spec.layers[1], arrangement="pre_norm")
    with pytest.raises(ConfigError, match="streams"):
        dataclasses.replace(spec, layers=(spec.layers[0], plain, spec.layers[2])).validate()


def test_a_mixer_of_branches_gets_one_cache_view_a_branch():
    """The cache on the CPU: a layer whose mixer asks for two things (keys and values; a state) beside layers that ask for one."""
    from titan_b200.cache import SequenceCache
    from titan_b200.cache.groups import KVGroup, StateGroup
    from titan_b200.config import config_from_dict
    from titan_b200.parts import build_block
    spec = config_from_dict(make_config("odd")).to_model_spec()
    needs = [build_block(l).mixer.cache_need() for l in spec.layers]
    assert isinstance(needs[1], tuple) and [n.kind for n in needs[1]] == ["kv", "state"]
    assert needs[1][0].window == 7 and needs[2][0].window is None                 # kept first tokens: every key stays, the window is a mask
    cache = SequenceCache(needs, 256, 3, 128, torch.float32, "cpu")
    one = cache.view_for_layer(0)
    assert isinstance(one[0], StateGroup)
    two = cache.view_for_layer(1)
    assert isinstance(two, tuple) and isinstance(two[0][0], KVGroup) and isinstance(two[1][0], StateGroup)
    assert two[0][0].ring_rows == 64 and cache.view_for_layer(2)[0][0].ring_rows == 0
    s = cache.alloc_slot()
    cache.reserve({s: 100})
    cache.commit(s, 100)
    cache.check()
    cache.free_slot(s)
    cache.check()


def test_a_folder_of_random_weights_is_written_and_read_back(tmp_path):
    from titan_b200.config import config_from_dict, load_config
    from titan_b200.parts import declare_weights
    from titan_b200.weights import FolderWeights, write_model_folder
    folder = write_model_folder(str(tmp_path / "m"), config_from_dict(make_config("mix")), seed=4)
    cfg = load_config(folder)
    declared = declare_weights(cfg.to_model_spec())
    source = FolderWeights(folder, declared, torch.float32, "cpu")
    by_name = {w.name: w for w in declared}
    assert source.get(by_name["l0.hc2.mix"]).shape == (2, 2) and source.get(by_name["l0.mix.right.v.conv"]).shape == (48, 3)
    assert abs(float(source.get(by_name["l0.hc1.in"]).mean()) - 0.5) < 0.5


def test_the_second_sublayers_small_tensors_may_be_in_the_file_of_a_layer_without_one(tmp_path):
    from titan_b200.config import load_config
    from titan_b200.parts import declare_weights
    from titan_b200.weights import FolderWeights, WeightError
    cfg = make_config("mix")
    weights = {k: v.to(torch.bfloat16) for k, v in random_weights(cfg, 2).items()}
    weights["l1.norm2"] = torch.ones(cfg["width"], dtype=torch.bfloat16)
    folder = write_folder(str(tmp_path / "m"), cfg, weights)
    spec = load_config(folder).to_model_spec()
    FolderWeights(folder, declare_weights(spec), torch.float32, "cpu", spec.ignorable_tensors)
    with pytest.raises(WeightError):
        FolderWeights(folder, declare_weights(spec), torch.float32, "cpu")


# --------------------------------------------------------------------------- #
# the plain implementation's own mechanisms, against cases worked by hand
# --------------------------------------------------------------------------- #
def test_plain_window_and_kept_tokens():
    assert [j for j in range(10) if P.sees(9, j, 3, 2)] == [0, 1, 7, 8, 9]
    assert [j for j in range(10) if P.sees(9, j, 3, 0)] == [7, 8, 9]
    assert [j for j in range(4) if P.sees(2, j, None, 0)] == [0, 1, 2]
    assert [j for j in range(10) if P.sees(3, j, 2, 5)] == [0, 1, 2, 3]           # kept tokens are still causal


def test_plain_rotation_pairs_neighbours_and_keeps_the_rest():
    x = np.arange(12, dtype=np.float64).reshape(1, 1, 12) + 1
    y = P.rotate_adjacent(np.repeat(x, 2, 0), np.array([0.0, 3.0]), 4, 100.0)
    assert np.allclose(y[0], x[0]) and np.allclose(y[1, 0, 4:], x[0, 0, 4:])
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert np.allclose(y[1, 0, :4], [1 * np.cos(a0) - 2 * np.sin(a0), 2 * np.cos(a0) + 1 * np.sin(a0), 3 * np.cos(a1) - 4 * np.sin(a1), 4 * np.cos(a1) + 3 * np.sin(a1)])


def test_plain_convolution_puts_the_last_tap_on_the_current_token():
    x = np.array([[1.0], [10.0], [100.0]])
    assert np.allclose(P.short_conv(x, np.array([[3.0, 2.0]]))[:, 0], [2.0, 23.0, 230.0])


def test_plain_sink_counts_once_and_has_no_value():
    """One token: the softmax weight of its own key is e^s / (e^s + e^sink)."""
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "rot": {"base": 10.0, "dims": 2}, "scale": 1.0}
    w = {"q": np.eye(2), "k": np.eye(2), "v": np.array([[3.0, 0.0], [0.0, 4.0]]), "sink": np.array([0.7]), "g": np.zeros((2, 2)), "o": np.eye(2)}
    h = np.array([[1.0, 1.0]])
    weight = np.exp(2.0) / (np.exp(2.0) + np.exp(0.7))
    v = np.array([3.0, 4.0]) / np.sqrt(12.5 + 1e-6)
    assert np.allclose(P.windowed_sink_attention(h, w, m, 1e-6), 0.5 * weight * v)


def test_plain_delta_rule_replaces_what_a_key_held():
    """With beta = 1 and no decay, writing a second value under the same unit key leaves only the second."""
    S = np.zeros((2, 2))
    k = np.array([1.0, 0.0])
    for v in (np.array([5.0, 6.0]), np.array([-1.0, 2.0])):
        u = 1.0 * (v - S.T @ k)
        S = S + np.outer(k, u)
    assert np.allclose(S.T @ k, [-1.0, 2.0])


def test_plain_mlstm_first_token_by_hand():
    m = {"heads": 1, "dim": 1, "vdim": 1, "gate_cap": 5.0}
    z = np.zeros((1, 1))
    w = {"q": np.ones((1, 1)), "k": np.ones((1, 1)), "v": np.ones((1, 1)), "g": z, "o": np.ones((1, 1)), "norm": np.ones(1),
         "i": z, "f": z, "i.b": np.array([-2.0]), "f.b": np.array([1.0])}
    # i = 5 tanh(-0.4) < 0, so m stays max(f + 0, i) = f = logsigmoid(5 tanh(0.2)): the maximum starts at zero, not at minus infinity
    f = -np.log1p(np.exp(-5 * np.tanh(0.2)))
    i = 5 * np.tanh(-0.4)
    S = np.exp(i - f) * 2.0 * 2.0
    n = np.exp(i - f) * 2.0
    o = S * 2.0 / (max(abs(n * 2.0), np.exp(-f)) + 1e-6)
    want = 0.5 * o / np.sqrt(o * o + 1e-6)
    assert np.allclose(P.mlstm(np.array([[2.0]]), w, m, 1e-6), want)
