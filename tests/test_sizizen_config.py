"""The Sizizen configuration reader and the description it builds (no device needed)."""
import copy

import pytest

from sizizen_helpers import CONFIG_A, CONFIG_B
from purhie_b200.config import ConfigError, ModelConfig, registered_architectures, registered_parts
from purhie_b200.weights import expected_tensors


def test_the_architecture_and_its_parts_are_registered():
    assert "Sizizen" in registered_architectures()
    assert {"layernorm", "none"} <= set(registered_parts("norm"))
    assert {"attention", "gated_linear_attention", "side_by_side"} <= set(registered_parts("mixer"))
    assert {"swiglu", "mlp", "routed_glu"} <= set(registered_parts("feed_forward"))


def test_the_description_follows_the_layer_list():
    cfg = ModelConfig.from_dict(CONFIG_A)
    assert cfg.architecture == "Sizizen"
    spec = cfg.model_spec()
    kinds = [(l["parts"]["mixer"]["kind"], l["parts"].get("feed_forward", {}).get("kind")) for l in spec["layers"]]
    assert kinds == [("side_by_side", "swiglu"), ("side_by_side", "routed_glu"), ("side_by_side", None), ("side_by_side", "routed_glu")]
    for l in spec["layers"]:
        assert l["arrangement"] == "sandwich_norm" and l["params"]["residual_factor"] == 1.0
        assert l["parts"]["mixer_norm"]["kind"] == "none" and l["parts"]["mixer_post_norm"]["kind"] == "layernorm"
        assert "bias" not in l["parts"]["mixer_post_norm"]["params"]["names"]
    m = spec["layers"][3]["parts"]["mixer"]["params"]
    a, r = m["left"]["params"], m["right"]["params"]
    assert m["factor"] == 0.5 and m["left"]["kind"] == "attention" and m["right"]["kind"] == "gated_linear_attention"
    assert (a["num_heads"], a["num_kv_heads"], a["head_dim"], a["value_dim"], a["chunk"], a["scale"]) == (2, 1, 24, 16, 16, 0.15)
    assert a["bias"] is True and a["qk_norm_eps"] == 1e-6 and a["window"] is None
    assert a["position"]["params"] == {"theta": 1e6, "n_rot": 12, "max_position": 65536, "pairing": "half"}
    assert (r["num_heads"], r["head_dim"], r["value_dim"], r["tau"], r["decay_rank"]) == (4, 8, 8, 2.0, 8)
    f = spec["layers"][1]["parts"]["feed_forward"]["params"]
    assert (f["experts"], f["top"], f["gated"], f["activation"]) == (6, 2, False, "relu2")
    assert f["scoring"] == {"kind": "sigmoid", "groups": 3, "keep": 2}
    assert f["shared"]["kind"] == "mlp" and f["shared"]["params"]["intermediate_size"] == 24
    assert spec["final_norm"]["kind"] == "layernorm" and "scale" not in spec["embedding"]["params"]


def test_the_tensor_list_has_every_name_with_its_shape():
    t = expected_tensors(CONFIG_A)
    assert tuple(t["embed"].shape) == (80, 48) and tuple(t["head"].shape) == (80, 48) and tuple(t["final.norm"].shape) == (48,)
    assert tuple(t["l0.mix.left.q"].shape) == (64, 48) and tuple(t["l0.mix.left.q.b"].shape) == (64,)
    assert tuple(t["l0.mix.left.k"].shape) == (32, 48) and tuple(t["l0.mix.left.v"].shape) == (16, 48) and tuple(t["l0.mix.left.v.b"].shape) == (16,)
    assert tuple(t["l0.mix.left.q.norm"].shape) == (16,) and tuple(t["l0.mix.left.o"].shape) == (48, 32)
    assert tuple(t["l0.mix.right.q"].shape) == (16, 48) and tuple(t["l0.mix.right.v"].shape) == (32, 48) and tuple(t["l0.mix.right.g"].shape) == (32, 48)
    assert tuple(t["l0.mix.right.a1"].shape) == (6, 48) and tuple(t["l0.mix.right.a2"].shape) == (16, 6) and tuple(t["l0.mix.right.a2.b"].shape) == (16,)
    assert tuple(t["l0.mix.right.norm"].shape) == (16,) and tuple(t["l0.mix.right.o"].shape) == (48, 32)
    assert tuple(t["l0.mix.left.out"].shape) == (48,) and tuple(t["l0.mix.right.out"].shape) == (48,)
    assert tuple(t["l1.mlp.router"].shape) == (6, 48) and tuple(t["l1.mlp.correction"].shape) == (6,)
    assert tuple(t["l1.mlp.e5.up"].shape) == (16, 48) and tuple(t["l1.mlp.e5.down"].shape) == (48, 16) and "l1.mlp.e0.gate" not in t
    assert tuple(t["l1.mlp.shared.up"].shape) == (24, 48) and tuple(t["l0.mlp.gate"].shape) == (64, 48)
    assert "l2.norm2" not in t and "l2.mlp.up" not in t and not any(n.endswith("norm1.b") for n in t)
    # without `rank` the two matrices of the decay are taken as they are stored
    bare = copy.deepcopy(CONFIG_A)
    del bare["layers"][0]["mixer"]["right"]["rank"]
    t = expected_tensors(bare)
    assert tuple(t["l0.mix.right.a1"].shape) == (-1, 48) and tuple(t["l0.mix.right.a2"].shape) == (16, -1)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="serial"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("mask"), "mask"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_a_configuration_that_does_not_fit_is_refused_by_name(change, word):
    c = copy.deepcopy(CONFIG_A)
    change(c)
    with pytest.raises(ConfigError) as e:
        ModelConfig.from_dict(c)
    assert word in str(e.value)


def test_a_random_model_folder_of_this_design_is_written_and_passes_the_folder_check(tmp_path):
    from purhie_b200.config import load_config
    from purhie_b200.weights import check_model_folder, list_tensors, write_random_model
    write_random_model(str(tmp_path), CONFIG_B, seed=3, std=0.05, scale_low=0.8, scale_high=1.2, dtype="bfloat16")
    check_model_folder(str(tmp_path))
    names = {t["name"]: t for t in list_tensors(str(tmp_path))}
    assert set(names) == set(expected_tensors(CONFIG_B))
    assert names["l1.mix.right.a2"]["shape"] == [80, 7] and names["l2.mlp.correction"]["shape"] == [9]
    assert load_config(str(tmp_path)).to_dict()["layers"] == CONFIG_B["layers"]


def test_a_size_that_only_a_folder_gives_cannot_be_drawn_at_random(tmp_path):
    from purhie_b200.native import InferenceError
    from purhie_b200.weights import write_random_model
    bare = copy.deepcopy(CONFIG_B)
    del bare["layers"][1]["mixer"]["right"]["rank"]
    with pytest.raises(InferenceError) as e:
        write_random_model(str(tmp_path), bare, seed=1)
    assert "a1" in str(e.value) or "rank" in str(e.value) or "stored" in str(e.value)
