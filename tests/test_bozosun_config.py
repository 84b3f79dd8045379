"""The Bozosun configuration reader and the description it builds (no device needed)."""
import copy

import pytest

from bozosun_helpers import CONFIG_A, CONFIG_B, attention, config, dense, mamba, moe, rot
from purhie_b200.config import ConfigError, ModelConfig, registered_architectures, registered_parts
from purhie_b200.weights import expected_tensors


def test_the_architecture_and_its_parts_are_registered():
    assert "Bozosun" in registered_architectures()
    assert "layernorm" in registered_parts("norm")
    assert {"attention", "mamba1"} <= set(registered_parts("mixer"))
    assert {"swiglu", "routed_glu"} <= set(registered_parts("feed_forward"))
    assert "sandwich_norm" in registered_parts("arrangement")


def test_the_description_follows_the_layer_list():
    cfg = ModelConfig.from_dict(CONFIG_B)
    assert cfg.architecture == "Bozosun"
    spec = cfg.model_spec()
    kinds = [(l["parts"]["mixer"]["kind"], l["parts"].get("feed_forward", {}).get("kind")) for l in spec["layers"]]
    assert kinds == [("mamba1", None), ("attention", "routed_glu"), ("attention", "swiglu"), ("attention", None),
                     ("attention", "routed_glu"), ("attention", "swiglu")]
    assert all(l["arrangement"] == "sandwich_norm" and l["params"]["residual_factor"] == 1.0 for l in spec["layers"])
    mixes = [l["parts"]["mixer"]["params"].get("value_mix") for l in spec["layers"]]
    assert mixes == [None, None, "first", None, "blend", "blend"]          # mixing starts at the first layer that asks
    a = spec["layers"][4]["parts"]["mixer"]["params"]
    assert (a["num_heads"], a["num_kv_heads"], a["head_dim"], a["value_dim"]) == (6, 2, 24, 40)
    assert a["position"]["params"]["pairing"] == "interleaved" and a["position"]["params"]["scaling"]["kind"] == "yarn"
    assert spec["layers"][3]["parts"]["mixer"]["params"]["position"] is None
    assert spec["layers"][1]["parts"]["mixer"]["params"]["position"]["params"]["n_rot"] == 12
    f = spec["layers"][4]["parts"]["feed_forward"]["params"]
    assert (f["experts"], f["top"], f["activation"]["limit"]) == (7, 7, 2.0)
    assert spec["embedding"]["params"]["scale"] == 1.0 and spec["final_norm"]["kind"] == "layernorm"


def test_the_tensor_list_has_every_name_with_its_shape():
    t = expected_tensors(CONFIG_A)
    assert tuple(t["embed"].shape) == (96, 48) and tuple(t["head"].shape) == (96, 48)
    assert tuple(t["l0.mix.q"].shape) == (64, 48) and tuple(t["l0.mix.v"].shape) == (16, 48) and tuple(t["l0.mix.o"].shape) == (48, 32)
    assert tuple(t["l2.mix.vmix"].shape) == () and "l0.mix.vmix" not in t
    assert tuple(t["l1.mix.in"].shape) == (128, 48) and tuple(t["l1.mix.x"].shape) == (5 + 16, 64)
    assert tuple(t["l1.mix.conv"].shape) == (64, 3) and tuple(t["l1.mix.A_log"].shape) == (64, 8) and tuple(t["l1.mix.dt"].shape) == (64, 5)
    assert tuple(t["l1.mlp.router"].shape) == (5, 48) and tuple(t["l1.mlp.e4.down"].shape) == (48, 24)
    for i in range(4):
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            assert tuple(t[f"l{i}.{n}"].shape) == (48,) and tuple(t[f"l{i}.{n}.b"].shape) == (48,)
    b = expected_tensors(CONFIG_B)
    assert "l0.norm2" not in b and "l0.mlp.gate" not in b and "l3.norm2b.b" not in b       # layers without a feed-forward


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=12), "v_mix"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][1]["mixer"].pop("state"), "state"),
])
def test_a_configuration_that_does_not_fit_is_refused_by_name(change, word):
    c = copy.deepcopy(CONFIG_A)
    change(c)
    with pytest.raises(ConfigError) as e:
        ModelConfig.from_dict(c)
    assert word in str(e.value)


def test_other_architectures_are_still_read_by_their_list_of_names():
    from helpers import TINY_A
    assert ModelConfig.from_dict(TINY_A).architecture == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError):
        ModelConfig.from_dict({"vocab": 3})


def test_a_random_model_folder_of_this_design_is_written_and_passes_the_folder_check(tmp_path):
    from purhie_b200.config import load_config
    from purhie_b200.weights import check_model_folder, list_tensors, write_random_model
    write_random_model(str(tmp_path), CONFIG_B, seed=3, std=0.05, scale_low=0.8, scale_high=1.2, dtype="bfloat16")
    check_model_folder(str(tmp_path))
    names = {t["name"]: t for t in list_tensors(str(tmp_path))}
    assert set(names) == set(expected_tensors(CONFIG_B))
    assert names["l4.mix.vmix"]["shape"] == [] and names["l0.mix.A_log"]["shape"] == [56, 20]
    assert load_config(str(tmp_path)).to_dict()["layers"] == CONFIG_B["layers"]
