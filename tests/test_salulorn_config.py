"""The Salulorn configuration on the host, without a GPU: reading config.json, what it refuses, the model spec it becomes
(the loop as a schedule), and the check of a checkpoint against it."""
import copy

import pytest

from salulorn_cases import CASES, CASE_A, CASE_B, CASE_D, random_weights, tensor_shapes, write_model


def test_registered_and_chosen_by_name():
    from fastgguf_b200.config import SalulornConfig
    from fastgguf_b200.registry import config_from_dict, registered_architectures
    assert "Salulorn" in registered_architectures()
    cfg = config_from_dict(CASE_A[0])
    assert isinstance(cfg, SalulornConfig) and cfg.architecture == "Salulorn"
    assert cfg.to_dict() == CASE_A[0]
    d = cfg.describe()
    assert d["hidden_size"] == 96 and d["vocab_size"] == 211 and d["num_hidden_layers"] == 4 and d["layer_runs"] == 8
    assert d["layer_kinds"] == ["gla+dense", "attention+dense", "latent_attention+none", "gla+dense"]
    # per run of a layer: the attention layer's keys and values and the latent layer's latent, three passes each
    assert d["kv_bytes_per_token"]["bfloat16"] == 2 * 3 * (2 * (24 + 40) + 40 + 8)
    conv_state = 3 * (4 * 24 + 2 * (24 + 40))
    assert d["state_bytes_per_sequence"] == 4 * (3 * 16 * 24 + 2 * 32 * 16 + 3 * conv_state)


def test_the_loop_becomes_a_schedule():
    from fastgguf_b200.registry import config_from_dict
    spec = config_from_dict(CASE_A[0]).spec_json()
    assert [(r["layer"], r.get("reenter", False)) for r in spec["schedule"]] == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True),
                                                                     (2, False), (3, False)]
    assert spec["reentry"]["kind"] == "concat_linear" and spec["reentry"]["tensors"] == {"weight": "loop.in"}
    once = config_from_dict(CASE_D[0]).spec_json()
    assert [(r["layer"], r.get("reenter", False)) for r in once["schedule"]] == [(0, False), (1, True)]
    none = config_from_dict(CASE_B[0]).spec_json()
    assert "reentry" not in none and [r["layer"] for r in none["schedule"]] == [0, 1, 2, 3, 4] and not any("reenter" in r for r in none["schedule"])


def test_spec_follows_the_file():
    from fastgguf_b200.registry import config_from_dict
    spec = config_from_dict(CASE_A[0]).spec_json()
    kinds = [(l["block"], l["mixer"]["kind"], (l["feed_forward"] or {}).get("kind")) for l in spec["layers"]]
    assert kinds == [("parallel", "gated_linear_attention", "swiglu"), ("parallel", "sink_attention", "swiglu"),
                     ("parallel", "latent_attention", None), ("parallel", "gated_linear_attention", "swiglu")]
    assert all("feed_forward_norm" not in l or l["feed_forward_norm"] is None for l in spec["layers"])
    a = spec["layers"][1]["mixer"]["params"]
    assert (a["window"], a["n_kv_heads"], a["head_dim"], a["v_head_dim"], a["scale"], a["softcap"], a["conv_taps"]) == (9, 2, 24, 40, 0.3, 20.0, 4)
    assert a["position"]["params"] == {"head_dim": 24, "theta": 10000.0, "rotary_dim": 8, "layout": "adjacent", "scaling": None}
    assert a["bias"] and a["sink"] and a["qk_norm"] == "whole" and a["eps"] == 1e-6
    m = spec["layers"][2]["mixer"]["params"]
    assert (m["rot_dim"], m["kv_rank"], m["q_rank"], m["head_dim"], m["v_head_dim"]) == (8, 40, 48, 16, 24)
    assert m["position"]["params"]["scaling"] == {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64.0,
                                                   "beta_fast": 8.0, "beta_slow": 1.0}
    g = spec["layers"][0]["mixer"]["params"]
    assert g["tau"] == 4.0 and g["q_scale"] == 0.25 and "decay_rank" not in g
    plain = config_from_dict(CASE_B[0]).spec_json()["layers"]
    p = plain[2]["mixer"]["params"]
    assert p["window"] == 0 and p["softcap"] == 0.0 and p["conv_taps"] == 0 and p["position"] is None and p["n_kv_heads"] == 2
    assert plain[1]["mixer"]["params"]["position"]["params"]["scaling"] is None
    assert spec["head"]["tensors"]["weight"] == "head" and spec["embedding"]["tensors"]["weight"] == "embed"


def test_python_spec_round_trip():
    from fastgguf_b200.engine.spec import ModelSpec
    from fastgguf_b200.registry import config_from_dict
    j = config_from_dict(CASE_A[0]).spec_json()
    again = ModelSpec.from_json(j).to_json()
    assert again["schedule"] == j["schedule"] and again["reentry"] == j["reentry"]
    assert again["layers"][2]["feed_forward"] is None and again["layers"][0]["feed_forward_norm"] is None


def broken(path, value):
    d = copy.deepcopy(CASE_A[0])
    node = d
    for k in path[:-1]:
        node = node[k]
    if value is KeyError:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return d


@pytest.mark.parametrize("path,value,needle", [
    (["vocab"], KeyError, "vocab"), (["width"], 0, "positive"), (["norm", "eps"], 0.0, "eps"), (["norm"], KeyError, "norm"),
    (["layers", 0, "type"], "conv", "not known"), (["layers", 0, "mixer", "tau"], 0.0, "tau"),
    (["layers", 1, "mixer", "rot", "dims"], 7, "dims"), (["layers", 1, "mixer", "rot", "dims"], 26, "dims"),
    (["layers", 1, "mixer", "kv_heads"], 3, "multiple"), (["layers", 1, "mixer", "mask", "size"], 0, "size"),
    (["layers", 1, "mixer", "softcap"], -1.0, "softcap"), (["layers", 2, "mixer", "rot_dim"], 7, "rot_dim"),
    (["layers", 2, "mixer", "rot", "dims"], 4, "rot_dim"), (["layers", 2, "mixer", "rot", "scaling", "factor"], 0.0, "positive"),
    (["layers", 2, "mixer", "kv_rank"], KeyError, "kv_rank"), (["layers", 0, "mlp", "kind"], "moe", "not known"),
    (["layers", 0, "mlp", "ff"], 0, "ff"), (["loop", "stop"], 5, "stop"), (["loop", "start"], 3, "start"), (["loop", "times"], 0, "times"),
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
    for name, case in CASES.items():
        declared = expected_tensors(config_from_dict(case[0]))
        want = tensor_shapes(case)
        assert sorted(declared) == sorted(want), name
        for k, v in declared.items():
            # the inner size of a decay pair is left to the checkpoint
            assert all(a == b or a == -1 for a, b in zip(v["shape"], want[k])) and len(v["shape"]) == len(want[k]), (name, k)
    W = random_weights(CASE_A, 1)
    good = write_model(tmp_path / "good", CASE_A, W)
    assert len(check_weights(config_from_dict(CASE_A[0]), model_dir=good)) == len(W)
    bad = dict(W)
    del bad["l1.mix.sink"]
    bad["l2.mlp.up"] = W["l0.mlp.up"]                 # a layer without a feed-forward has no tensors for one
    bad["l3.mix.g"] = W["l3.mix.g"][:, :-1].contiguous()
    with pytest.raises(WeightError) as e:
        check_weights(config_from_dict(CASE_A[0]), model_dir=write_model(tmp_path / "bad", CASE_A, bad))
    assert e.value.missing == ["l1.mix.sink"] and e.value.unexpected == ["l2.mlp.up"] and "l3.mix.g" in e.value.wrong[0]


def test_random_model_folder_needs_every_size(tmp_path):
    """The framework's own writer of seeded random folders: with the decay pair's inner size in the file it works; without,
    it says which size is missing."""
    from fastgguf_b200.registry import config_from_dict, config_from_dir
    from fastgguf_b200.weights import check_weights, write_random_model
    cfg = copy.deepcopy(CASE_B[0])
    with pytest.raises(Exception) as e:
        write_random_model(config_from_dict(cfg), 5, str(tmp_path / "open"))
    assert "checkpoint" in str(e.value)
    cfg["layers"][3]["mixer"]["decay_rank"] = 8
    d = write_random_model(config_from_dict(cfg), 5, str(tmp_path / "r"))
    again = config_from_dir(d)
    assert again.describe()["layer_kinds"] == config_from_dict(cfg).describe()["layer_kinds"]
    check_weights(again, model_dir=d)


def test_kernel_libraries_by_model():
    from fastgguf_b200 import capi
    from fastgguf_b200.registry import config_from_dict
    spec = config_from_dict(CASE_B[0]).spec_json()
    assert capi.kernel_modules_for(spec, capi.FG_BF16) == ("core", "tc", "mix")
    assert capi.kernel_modules_for(spec, capi.FG_F32) == ("core", "mix")
