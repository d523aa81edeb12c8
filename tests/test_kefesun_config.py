"""The Kefesun configuration class: what it reads, what it refuses, and the model it
describes (no GPU needed)."""
import copy

import pytest

from janas_b200.config import ConfigError, KefesunConfig, config_from_dict, known_architectures
from janas_b200.weights import expected_tensors
from kefesun_models import CONFIGS, tensor_shapes


def test_registered():
    assert "Kefesun" in known_architectures()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_list_matches_the_design(name):
    c = config_from_dict(CONFIGS[name])
    assert isinstance(c, KefesunConfig)
    got = {n: tuple(s.shape) for n, s in expected_tensors(c.to_model_spec()).items() if not s.optional}
    assert got == {n: tuple(s) for n, s in tensor_shapes(CONFIGS[name]).items()}


def test_spec_describes_the_layers():
    c = config_from_dict(CONFIGS["KA"])
    assert c.taps == 3 and c.embedding_scale == 8.0
    spec = c.to_model_spec()
    assert spec.tie_embeddings and spec.embedding_scale == 8.0 and spec.embedding_name == "embed"
    assert [e.layer for e in spec.run_order] == [0, 1, 2]
    l0, l1, l2 = spec.layers
    for l in spec.layers:
        assert l.block == "result_norm" and l.mixer_norm is None and l.ffn_norm is None
        assert l.post_mixer_norm.kind == "layernorm" and l.post_mixer_norm.get("names")["bias"] is None
        assert l.block_params["conv_taps"] == 3
    m = l0.mixer
    assert m.kind == "sink_attention" and m.get("window") == 37 and m.get("keep_first") == 5
    assert m.get("score_bias") is True and m.get("bias") is True and m.get("out_bias") is False
    assert m.get("qk_norm_eps") == 1e-6 and m.get("v_head_dim") == 24
    assert m.get("position").kind == "rope_neox" and m.get("position").get("rotary_dim") == 8
    assert l1.mixer.kind == "mingru" and l1.mixer.get("width") == 48
    f = l0.feed_forward
    assert f.kind == "routed" and f.get("experts") == 6 and f.get("identity") == 2 and f.get("top") == 3
    assert f.get("groups") == 4 and f.get("group_keep") == 2 and f.get("scale") == 1.7
    assert f.get("shared_ff") == 24 and f.get("activation") == "relu2" and f.get("correction") is True
    assert l2.feed_forward.get("shared_ff") == 0
    spec.validate()
    # what a layer leaves out is off: no window, no kept tokens, no rotation, no convolution
    kb = config_from_dict(CONFIGS["KB"]).to_model_spec()
    assert kb.layers[1].mixer.get("window") == 0 and kb.layers[1].mixer.get("keep_first") == 0
    assert kb.layers[1].mixer.get("position") is None
    assert kb.layers[2].feed_forward is None and kb.layers[2].post_ffn_norm is None
    assert config_from_dict(CONFIGS["KE"]).to_model_spec().layers[0].block_params["conv_taps"] == 0


def test_round_trip():
    for name, c in CONFIGS.items():
        d = config_from_dict(c).to_dict()
        assert config_from_dict(d).to_dict() == d
        assert d["vocab"] == c["vocab"] and d["width"] == c["width"]
        for a, b in zip(d["layers"], c["layers"]):
            assert a["type"] == b["type"]
            for k, v in b["mixer"].items():
                assert a["mixer"][k] == v


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0].update(type="conv"), "mixers"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=18), "at most"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "positive"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(keep=5), "keep"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda d: d["layers"][1]["mixer"].update(width=0), "width"),
    (lambda d: d["canon"].update(taps=0), "taps"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d["layers"][0]["mixer"].update(dim=600), "512"),
])
def test_refusals(change, word):
    d = copy.deepcopy(CONFIGS["KA"])
    change(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)
