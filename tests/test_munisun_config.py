"""The Munisun configuration class: what it reads, what it refuses, and the model it
describes (no GPU needed)."""
import copy

import pytest

from janas_b200.config import ConfigError, MunisunConfig, config_from_dict, known_architectures
from janas_b200.weights import expected_tensors
from munisun_models import CONFIGS, tensor_shapes


def test_registered():
    assert "Munisun" in known_architectures()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_list_matches_the_design(name):
    c = config_from_dict(CONFIGS[name])
    assert isinstance(c, MunisunConfig)
    got = {n: tuple(s.shape) for n, s in expected_tensors(c.to_model_spec()).items() if not s.optional}
    assert got == {n: tuple(s) for n, s in tensor_shapes(CONFIGS[name]).items()}


def test_spec_describes_the_layers():
    c = config_from_dict(CONFIGS["MA"])
    assert c.side_dim == 8 and c.embedding_scale == 4.0
    spec = c.to_model_spec()
    assert not spec.tie_embeddings and spec.head_name == "head" and spec.embedding_name == "embed"
    assert spec.token_table_name == "side.embed" and spec.token_table_width == 16
    assert spec.final_norm.kind == "rmsnorm" and spec.final_norm.get("one_plus") is True
    assert [e.layer for e in spec.run_order] == [0, 1]
    l0, l1 = spec.layers
    for i, l in enumerate(spec.layers):
        assert l.block == "sandwich" and l.mixer.kind == "pair"
        for n in (l.mixer_norm, l.post_mixer_norm, l.ffn_norm, l.post_ffn_norm):
            assert n.kind == "rmsnorm" and n.get("one_plus") is True and n.get("names")["weight"] == ""
        ts = l.block_params["token_side"]
        assert ts["dim"] == 8 and ts["col0"] == 8 * i and ts["eps"] == 1e-6
    m = l0.mixer
    assert m.get("join") == "sum" and m.get("left_scale") == 0.7 and m.get("right_scale") == 1.1
    a = m.get("left")
    assert a.kind == "sink_attention" and a.get("gate") is True and a.get("softcap") == 6.0
    assert a.get("qk_norm_eps") == 1e-6 and a.get("qk_unit_norm_eps") is None and a.get("conv_taps") is None
    pos = a.get("position")
    assert pos.kind == "rope_pairs" and pos.get("rotary_dim") == 8
    assert pos.get("scaling") == {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 24.0}
    r = m.get("right")
    assert r.kind == "mamba2" and r.get("heads") == 4 and r.get("state") == 8 and r.get("groups") == 2
    assert r.get("conv_taps") == 3 and r.get("norm_groups") == 2
    assert l0.feed_forward.kind == "swiglu" and l0.feed_forward.get("intermediate_size") == 96
    m = l1.mixer
    assert m.get("join") == "normed_mean" and m.get("eps") == 1e-6
    a = m.get("left")
    assert a.get("conv_taps") == 3 and a.get("qk_unit_norm_eps") == 1e-6 and a.get("gate") is None
    assert a.get("qk_norm_eps") is None and a.get("softcap") is None and a.get("position").get("scaling") is None
    r = m.get("right")
    assert r.kind == "decay_attention" and r.get("decay") == [0.5, 0.9, 0.99] and r.get("v_head_dim") == 24
    f = l1.feed_forward
    assert f.kind == "routed" and f.get("experts") == 6 and f.get("top") == 2 and f.get("gated") is True
    assert f.get("groups") == 3 and f.get("group_keep") == 2 and f.get("group_best") == 2
    assert f.get("score") == "sigmoid" and f.get("activation") == "silu" and f.get("correction") is True
    spec.validate()
    # what a model leaves out is off: no token input, no rotation, no feed-forward
    mb = config_from_dict(CONFIGS["MB"]).to_model_spec()
    assert mb.token_table_name == "" and "token_side" not in mb.layers[0].block_params
    assert mb.layers[0].mixer.get("left").get("position") is None
    assert mb.layers[0].feed_forward is None and mb.layers[0].post_ffn_norm is None


def test_round_trip():
    for name, c in CONFIGS.items():
        d = config_from_dict(c).to_dict()
        assert config_from_dict(d).to_dict() == d
        assert d["vocab"] == c["vocab"] and d["width"] == c["width"]
        for a, b in zip(d["layers"], c["layers"]):
            assert a["type"] == b["type"]
            if b["mlp"] is None or b["mlp"]["kind"] == "dense":
                assert a["mlp"] == b["mlp"]
            else:
                assert a["mlp"]["expert"] == b["mlp"]["expert"]
                for k, v in b["mlp"]["router"].items():         # groups left out are written as one group
                    assert a["mlp"]["router"][k] == v
            for side in ("left", "right"):
                for k, v in b["mixer"][side].items():
                    assert a["mixer"][side][k] == v, (name, side, k)


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0].update(type="attention"), "mixers"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "at most"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(groups=3), "groups"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(norm_groups=5), "norm_groups"),
    (lambda d: d["layers"][1]["mixer"]["right"].update(decay=[0.5, 0.9]), "decay"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(keep=5), "keep"),
    (lambda d: d["layers"][0]["mlp"].update(kind="relu"), "dense"),
    (lambda d: d["layers"][0]["mixer"].pop("right"), "right"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(dim=600), "512"),
])
def test_refusals(change, word):
    d = copy.deepcopy(CONFIGS["MA"])
    change(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)
