"""The Zirivik configuration on the host, without a GPU: reading config.json, what it refuses, the model spec it
becomes, and the check of a checkpoint against it."""
import copy
import json

import pytest

from zirivik_cases import CASES, CASE_A, CASE_B, random_weights, tensor_shapes, write_model


def test_registered_and_chosen_by_name():
    from fastgguf_b200.config import ZirivikConfig
    from fastgguf_b200.registry import config_from_dict, registered_architectures
    assert "Zirivik" in registered_architectures()
    cfg = config_from_dict(CASE_A)
    assert isinstance(cfg, ZirivikConfig) and cfg.architecture == "Zirivik"
    assert cfg.to_dict() == CASE_A
    d = cfg.describe()
    assert d["hidden_size"] == 96 and d["vocab_size"] == 211 and d["num_hidden_layers"] == 4
    assert d["layer_kinds"] == ["attention+dense", "retention+moe", "attention(shared)+none", "retention+dense"]
    assert d["parameters"] == sum(int(__import__("math").prod(s)) for s in tensor_shapes(CASE_A).values())
    assert d["state_bytes_per_sequence"] == 4 * (3 * 16 * 24 + 2 * 32 * 16)
    assert d["kv_bytes_per_token"]["bfloat16"] == 2 * 2 * (24 + 40)


def test_spec_follows_the_file():
    from fastgguf_b200.registry import config_from_dict
    spec = config_from_dict(CASE_B).spec_json()
    assert [r["cache_from"] for r in spec["schedule"]] == [None, None, 1, None]
    kinds = [(l["block"], l["mixer"]["kind"], (l["feed_forward"] or {}).get("kind")) for l in spec["layers"]]
    assert kinds == [("sandwich", "retention", "moe"), ("sandwich", "gqa_attention", "mlp"), ("sandwich", "gqa_attention", "moe"),
                     ("sandwich", "gqa_attention", "mlp")]
    a = spec["layers"][1]["mixer"]["params"]
    assert (a["window"], a["keep_first"], a["n_kv_heads"], a["head_dim"], a["v_head_dim"], a["scale"]) == (64, 70, 1, 48, 48, 0.15)
    assert a["position"] is None and not a["queries_only"]
    b = spec["layers"][2]["mixer"]
    assert b["params"]["queries_only"] and sorted(b["tensors"]) == ["o_proj.weight", "q_proj.weight"]
    assert spec["layers"][3]["mixer"]["params"]["window"] == 0          # no mask: every earlier key
    r = spec["layers"][0]["mixer"]["params"]
    assert r["decay"] == [0.99, 0.995, 0.999, 0.9995] and r["position"]["params"] == {
        "head_dim": 32, "theta": 500000.0, "rotary_dim": 32, "layout": "halves", "scaling": None}
    assert spec["layers"][0]["mixer_norm"]["params"] == {"size": 128, "eps": 1e-5, "offset": 1.0}
    assert spec["head"]["tensors"]["weight"] == spec["embedding"]["tensors"]["weight"] == "embed"
    assert spec["head"]["params"]["softcap"] == 50.0 and spec["embedding"]["params"]["scale"] == 8.0
    nofeed = __import__("fastgguf_b200.registry", fromlist=["x"]).config_from_dict(CASE_A).spec_json()["layers"][2]
    assert nofeed["feed_forward"] is None and "feed_forward_post_norm" not in nofeed and "mixer_post_norm" in nofeed


def test_python_spec_round_trip():
    from fastgguf_b200.engine.spec import ModelSpec
    from fastgguf_b200.registry import config_from_dict
    j = config_from_dict(CASE_A).spec_json()
    again = ModelSpec.from_json(j).to_json()
    assert again["layers"][2]["feed_forward"] is None and again["layers"][0]["mixer_post_norm"] == j["layers"][0]["mixer_post_norm"]
    assert again["schedule"] == j["schedule"]


def broken(path, value):
    d = copy.deepcopy(CASE_A)
    node = d
    for k in path[:-1]:
        node = node[k]
    if value is KeyError:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return d


@pytest.mark.parametrize("path,value,needle", [
    (["vocab"], KeyError, "vocab"), (["width"], 0, "positive"), (["norm", "eps"], 0.0, "eps"), (["logit_softcap"], -1.0, "logit_softcap"),
    (["layers", 0, "type"], "conv", "not known"), (["layers", 1, "mixer", "decay"], [0.9, 0.9], "decay"),
    (["layers", 1, "mixer", "rot", "dims"], 7, "dims"), (["layers", 1, "mixer", "rot", "dims"], 18, "dims"),
    (["layers", 0, "mixer", "kv_heads"], 3, "multiple"), (["layers", 2, "mixer", "kv_from"], 2, "earlier"),
    (["layers", 2, "mixer", "kv_from"], 1, "no keys and values"), (["layers", 2, "mixer", "vdim"], 24, "other sizes"),
    (["layers", 0, "mixer", "mask", "size"], 0, "size"), (["layers", 1, "mlp", "router", "top"], 6, "top"),
    (["layers", 1, "mlp", "expert", "limit"], 0.0, "limit"), (["layers", 0, "mlp", "kind"], "glu", "not known"),
    (["layers"], [], "layers"),
])
def test_what_the_reader_refuses(path, value, needle):
    from fastgguf_b200.config import ConfigError
    from fastgguf_b200.registry import config_from_dict
    with pytest.raises(ConfigError) as e:
        config_from_dict(broken(path, value))
    assert needle in str(e.value)


def test_weights_are_checked_against_the_configuration(tmp_path):
    from fastgguf_b200.registry import config_from_dict
    from fastgguf_b200.weights import WeightError, check_weights, expected_tensors
    for name, cfg in CASES.items():
        declared = expected_tensors(config_from_dict(cfg))
        assert {k: tuple(v["shape"]) for k, v in declared.items()} == tensor_shapes(cfg), name
    W = random_weights(CASE_A, 1)
    good = write_model(tmp_path / "good", CASE_A, W)
    assert len(check_weights(config_from_dict(CASE_A), model_dir=good)) == len(W)
    bad = dict(W)
    del bad["l1.mlp.e3.up"]
    bad["l2.mix.k"] = W["l0.mix.k"]                 # a layer that shares keys and values has no projections for them
    bad["l3.mix.g"] = W["l3.mix.g"][:, :-1].contiguous()
    with pytest.raises(WeightError) as e:
        check_weights(config_from_dict(CASE_A), model_dir=write_model(tmp_path / "bad", CASE_A, bad))
    assert e.value.missing == ["l1.mlp.e3.up"] and e.value.unexpected == ["l2.mix.k"] and "l3.mix.g" in e.value.wrong[0]


def test_random_model_folder_reads_back(tmp_path):
    """The framework's own writer of seeded random folders works for this architecture too."""
    from fastgguf_b200.registry import config_from_dict, config_from_dir
    from fastgguf_b200.weights import check_weights, write_random_model
    d = write_random_model(config_from_dict(CASE_B), 5, str(tmp_path / "r"))
    again = config_from_dir(d)
    assert again.describe()["layer_kinds"] == config_from_dict(CASE_B).describe()["layer_kinds"]
    check_weights(again, model_dir=d)


def test_kernel_libraries_by_model():
    from fastgguf_b200 import capi
    from fastgguf_b200.registry import config_from_dict
    from helpers import TINY_A
    spec = config_from_dict(CASE_B).spec_json()
    assert capi.kernel_modules_for(spec, capi.FG_BF16) == ("core", "tc", "mix")
    assert capi.kernel_modules_for(spec, capi.FG_F32) == ("core", "mix")
    assert capi.kernel_modules_for(config_from_dict(CASES["c"]).spec_json(), capi.FG_BF16) == ("core", "tc", "attn", "mix")
    assert capi.kernel_modules_for(config_from_dict(TINY_A).spec_json(), capi.FG_BF16) == ("core", "tc")
