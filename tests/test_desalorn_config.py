"""The Desalorn design's configuration on the CPU: specs from the description, refusals, the declared tensors against the list
written out by hand, the size that a tensor's shape gives, the distance table's rows, and the plain router on hand-made numbers."""
import copy
import json
import math

import numpy as np
import pytest
import torch

from desalorn_cases import attention, latent, layer, make_config, model, moe, random_weights, retention, shapes_of
from helpers import write_folder
from plain import desalorn_plain as P
from titan_b200.config import ConfigError, config_from_dict, load_config


def test_specs_follow_the_description():
    cfg = make_config("mix")
    spec = config_from_dict(cfg).to_model_spec()
    assert spec.architecture == "Desalorn" and spec.hidden_size == 48 and spec.vocab_size == 97
    assert spec.embedding_scale == 3.0 and spec.lm_head == "head" and spec.final_norm.groups == 3
    assert [l.arrangement for l in spec.layers] == ["parallel"] * 3
    assert [l.mixer.kind for l in spec.layers] == ["attention", "retention", "latent_attention"]
    assert all(l.option("residual_mult") == 0.5 and l.mixer_norm.groups == 3 and l.feed_forward_norm is None for l in spec.layers)
    a, r, m = (l.mixer for l in spec.layers)
    assert a.option("softcap") == 5.0 and a.option("rel_bias") == ("rel", 8, 40.0) and a.option("head_mix") == "talk" and a.position.kind == "none"
    assert r.option("decay") == (0.9, 0.97, 0.995) and r.position.rotary_dim == 4 and r.position.pairing == "half"
    assert m.window == 20 and m.option("q_rank") == 12 and m.position.pairing == "adjacent" and spec.layers[2].feed_forward is None
    f = spec.layers[0].feed_forward
    assert (f.option("routing"), f.option("group_best"), f.option("renormalize"), f.option("shared_gate")) == ("sigmoid_all", 2, False, False)
    assert (f.option("groups"), f.option("keep"), f.option("shared_size")) == (4, 2, 40)
    one = config_from_dict(make_config("odd")).to_model_spec()
    assert one.embedding_scale is None and one.final_norm.groups == 1 and one.layers[0].feed_forward.option("shared_size") == 0


@pytest.mark.parametrize("name", ["mix", "odd", "wide"])
def test_declared_tensors_are_the_designs(name):
    from titan_b200.parts import declare_weights
    cfg = make_config(name)
    declared = {w.name: tuple(w.shape) for w in declare_weights(config_from_dict(cfg).to_model_spec())}
    assert declared == shapes_of(cfg)


def test_refusals():
    def broken(change):
        cfg = make_config("mix")
        change(cfg)
        with pytest.raises(ConfigError):
            config_from_dict(cfg)
    broken(lambda c: c["layers"][0].update(type="conv"))
    broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3))
    broken(lambda c: c["layers"][0]["mixer"].update(bias_max=3))              # the last row would be reached inside the first half
    broken(lambda c: c["layers"][0]["mixer"].pop("bias_rows"))                # neither a key nor a tensor gives the rows
    broken(lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 0.5]))
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10))
    broken(lambda c: c["layers"][2]["mixer"]["rot"].update(dims=3))
    broken(lambda c: c["layers"][2]["mixer"].pop("q_rank"))
    broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=5))           # more than the open groups hold
    broken(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="dense"))
    broken(lambda c: c["norm"].update(groups=5))
    broken(lambda c: c["norm"].update(eps=0))
    broken(lambda c: c.update(layers=[]))


def test_table_rows_come_from_the_tensor(tmp_path):
    cfg = make_config("odd")
    w = random_weights(cfg, 1)
    stripped = copy.deepcopy(cfg)
    for l in stripped["layers"]:
        l["mixer"].pop("bias_rows", None)
    folder = write_folder(str(tmp_path / "m"), stripped, {k: v.to(torch.bfloat16) for k, v in w.items()})
    spec = load_config(folder).to_model_spec()
    assert spec.layers[1].mixer.option("rel_bias") == ("rel", 5, 17.0) and spec.layers[3].mixer.option("rel_bias") == ("rel", 12, 300.0)


@pytest.mark.parametrize("rows,far", [(8, 40), (5, 17.0), (12, 300), (32, 128), (16, 1000), (2, 3), (1, 9), (16, 120.5)])
def test_rows_of_the_distance_table(rows, far):
    """The mixer's spread of the table by distance against the plain function, distance by distance, and the ends: the distance
    itself below half the rows, the last row from ``far`` on."""
    from titan_b200.parts.attention import distance_rows
    got = distance_rows(rows, far)
    assert len(got) == math.ceil(far) + 1
    if rows >= 2:
        assert got == [P.distance_bucket(n, rows, far) for n in range(len(got))]
        assert got[: rows // 2] == list(range(rows // 2)) and got[-1] == rows - 1
        assert all(b >= a for a, b in zip(got, got[1:]))
        assert P.distance_bucket(10 * math.ceil(far), rows, far) == rows - 1
    else:
        assert set(got) == {0}


def test_plain_router_on_hand_made_scores():
    """Two groups of three: the first holds the single best choice score, the second the better pair; the pair decides which
    group is open.  Negative choice scores in the open group still beat everything in the closed one, and the weights are the
    sigmoids without the correction."""
    logit = lambda p: math.log(p / (1 - p))
    s = [0.9, 0.1, 0.1, 0.6, 0.6, 0.2]
    z = np.array([[logit(p) for p in s]])
    ids, wts = P.route(z, np.zeros(6), 2, 2, 1)
    assert sorted(ids[0]) == [3, 4] and np.allclose(wts[0], 0.6)
    ids, wts = P.route(z, np.array([0.0, 0.0, 0.0, -2.0, -2.0, -2.0]), 2, 2, 1)        # corrections push the second group below zero ...
    assert sorted(ids[0]) == [0, 1]                                                    # ... and the first one opens
    ids, wts = P.route(z, np.array([-5.0, -5.0, -5.0, -2.0, -2.0, -2.0]), 3, 2, 1)     # every choice score negative: the open group still serves
    assert sorted(ids[0]) == [3, 4, 5] and np.allclose(sorted(wts[0]), [0.2, 0.6, 0.6])


def test_a_random_weights_folder_is_written_and_read_back(tmp_path):
    from titan_b200.weights import FolderWeights, write_model_folder
    from titan_b200.parts import declare_weights
    cfg = make_config("mix")
    folder = str(tmp_path / "m")
    write_model_folder(folder, config_from_dict(cfg), seed=4)
    again = load_config(folder)
    back = again.to_dict()
    back.pop("torch_dtype", None)                       # what the writer adds
    assert json.loads(json.dumps(back)) == json.loads(json.dumps(config_from_dict(cfg).to_dict()))
    declared = declare_weights(again.to_model_spec())
    source = FolderWeights(folder, declared, torch.float32, "cpu", [])
    by = {w.name: w for w in declared}
    assert tuple(source.get(by["l0.mix.talk"]).shape) == (4, 4) and tuple(source.get(by["l0.mix.rel"]).shape) == (8, 4)
