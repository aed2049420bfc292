"""Vosurax's configuration, model description, run order, checkpoint map and cache needs, without a GPU."""
from __future__ import annotations

import copy

import pytest

from liyab_b200.config import describe_config, slot, supported_architectures
from liyab_b200.status import LiyabError
from vosurax_models import CONFIG_A, CONFIG_C, CONFIG_D


def test_registered_and_found_by_its_own_key():
    assert "vosurax" in supported_architectures()
    assert describe_config(CONFIG_A)["architecture"] == "vosurax"


def test_every_size_and_constant_comes_from_the_file():
    d = describe_config(CONFIG_A)["spec"]
    assert d["embedding"]["vocab_size"] == 160 and d["embedding"]["size"] == 96 and not d["head"]["tied"]
    assert d["position"]["kind"] == "none"
    assert d["final_norm"] == {"kind": "rms_norm", "size": 96, "groups": 1, "eps": 1e-5, "gain_offset": 1.0}
    for layer, raw in zip(d["layers"], CONFIG_A["layers"]):
        assert layer["arrangement"] == "pre_norm"
        names = [s["name"] for s in layer["slots"]]
        assert names == (["mixer_norm", "mixer", "ff_norm", "feed_forward"] if raw["mlp"] else ["mixer_norm", "mixer"])
        m, r = slot(layer, "mixer"), raw["mixer"]
        if raw["type"] == "retention":
            assert m["kind"] == "matrix_memory" and m["recurrence"] == "fixed_decay" and m["decay"] == r["decay"]
            assert (m["n_head"], m["dim"], m["vdim"], m["rot_dims"], m["rot_base"]) == (r["heads"], r["dim"], r["vdim"], r["rot"]["dims"], r["rot"]["base"])
            assert abs(m["k_scale"] - r["dim"] ** -0.5) < 1e-15 and m["q_scale"] == 1.0 and m["gate"] == "silu" and not m["norm_gain"]
        else:
            assert m["kind"] == "branch_sum" and m["scale"] == 0.5 and [b["name"] for b in m["branches"]] == ["left", "right"]
            left, right = (b["part"] for b in m["branches"])
            a = r["left"]
            assert left["kind"] == "gated_attention" and left["qk_norm"] and left["bias"] and left["gate"] == "sigmoid"
            assert (left["n_head"], left["n_kv_head"], left["dim"], left["vdim"], left["scale"], left["chunk"]) == (
                a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["scale"], a["mask"]["size"])
            b = r["right"]
            assert right["kind"] == "matrix_memory" and right["recurrence"] == "gated" and right["gate_cap"] == b["gate_cap"]
            assert (right["n_head"], right["dim"], right["vdim"]) == (b["heads"], b["dim"], b["vdim"]) and abs(right["q_scale"] - b["dim"] ** -0.5) < 1e-15
        if raw["mlp"] and raw["mlp"]["kind"] == "moe":
            ff = slot(layer, "feed_forward")
            assert ff["kind"] == "routed" and (ff["experts"], ff["top"], ff["inner"]) == (raw["mlp"]["router"]["experts"], raw["mlp"]["router"]["top"], raw["mlp"]["expert"]["ff"])
            assert ff["shared_inner"] == raw["mlp"].get("shared", {}).get("ff", 0) and ff["score"] == "sigmoid" and not ff["renormalise"] and ff["weight_on"] == "input"
        elif raw["mlp"]:
            ff = slot(layer, "feed_forward")
            assert ff["kind"] == "dense" and ff["inner"] == raw["mlp"]["ff"] and ff["activation"] == "gelu_tanh" and not ff["bias"]
    # A branch without a mask sees every earlier key.
    c = describe_config(CONFIG_C)["spec"]
    assert slot(c["layers"][2], "mixer")["branches"][0]["part"]["chunk"] == 0


def test_a_stretch_runs_several_times_with_units_and_offsets_of_its_own():
    d = describe_config(CONFIG_A)["spec"]
    order = [(e["layer"], e["cache"], e.get("offset_row", -1)) for e in d["run_order"]]
    assert order == [(0, 0, -1), (1, 1, 0), (2, 2, -1), (1, 3, 1), (2, 4, -1), (1, 5, 2), (2, 6, -1), (3, 7, -1)]
    assert d["pass_offsets"] == 3
    # No stretch: every layer once, no offsets, and a file need not hold any.
    plain = describe_config(CONFIG_D)
    assert [(e["layer"], e["cache"]) for e in plain["spec"]["run_order"]] == [(0, 0), (1, 1), (2, 2)] and "pass_offsets" not in plain["spec"]
    assert "pass_offsets.weight" not in plain["checkpoint"]
    # A stretch from the first layer on, and one that runs once.
    c = copy.deepcopy(CONFIG_A)
    c["loop"] = dict(start=0, stop=4, times=1)
    assert [e.get("offset_row", -1) for e in describe_config(c)["spec"]["run_order"]] == [0, -1, -1, -1]


def test_checkpoint_map_joins_the_file_tensors():
    ck = describe_config(CONFIG_A)["checkpoint"]
    proj = ck["layers.0.mixer.proj.weight"]
    assert [s["name"] for s in proj["sources"]] == ["l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.g"]
    assert [s["shape"] for s in proj["sources"]] == [[48, 96], [48, 96], [72, 96], [72, 96]]
    left = ck["layers.1.mixer.left.proj.weight"]
    assert [s["name"] for s in left["sources"]] == ["l1.mix.left.q", "l1.mix.left.k", "l1.mix.left.v", "l1.mix.left.g"]
    assert [s["shape"][0] for s in left["sources"]] == [48, 24, 40, 80]
    assert [s["name"] for s in ck["layers.1.mixer.left.qkv_bias"]["sources"]] == ["l1.mix.left.q.b", "l1.mix.left.k.b", "l1.mix.left.v.b"]
    right = ck["layers.1.mixer.right.proj.weight"]
    assert [s["name"].rsplit(".", 1)[1] for s in right["sources"]] == ["q", "k", "v", "g", "i", "f"]
    assert [s["name"] for s in ck["layers.1.mixer.right.gate_bias"]["sources"]] == ["l1.mix.right.i.b", "l1.mix.right.f.b"]
    assert ck["layers.1.mixer.left_out.weight"]["sources"][0]["name"] == "l1.mix.left.out"
    experts = ck["layers.1.feed_forward.experts.gate_up.weight"]
    assert [s["name"] for s in experts["sources"]][:4] == ["l1.mlp.e0.gate", "l1.mlp.e0.up", "l1.mlp.e1.gate", "l1.mlp.e1.up"] and len(experts["sources"]) == 12
    assert len(ck["layers.1.feed_forward.experts.down.weight"]["sources"]) == 6
    assert "layers.2.ff_norm.weight" not in ck and "layers.3.feed_forward.shared.down.weight" not in ck
    assert ck["pass_offsets.weight"]["sources"][0] == {"name": "loop.step", "shape": [3, 96]}


@pytest.mark.parametrize("damage, text", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "retention, parallel"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("decay", [0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 5), "rot"),
    (lambda c: c["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["right"].__setitem__("gate_cap", 0.0), "gate_cap"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 7), "top"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "routed"), "dense, moe"),
    (lambda c: c["loop"].__setitem__("stop", 9), "stop"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configurations_are_refused(damage, text):
    c = copy.deepcopy(CONFIG_A)
    damage(c)
    with pytest.raises(LiyabError) as e:
        describe_config(c)
    assert text in str(e.value)
