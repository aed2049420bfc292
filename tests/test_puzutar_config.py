"""Puzutar's configuration, model description, checkpoint map and cache needs, without a GPU."""
from __future__ import annotations

import copy

import pytest

from liyab_b200.cache import CacheManager, KvNeed, StateNeed
from liyab_b200.config import describe_config, slot, supported_architectures
from liyab_b200.status import LiyabError
from puzutar_models import CONFIG_P, CONFIG_Q


def test_registered_and_found_by_its_own_key():
    assert "puzutar" in supported_architectures()
    assert describe_config(CONFIG_P)["architecture"] == "puzutar"


def test_every_size_comes_from_the_file():
    d = describe_config(CONFIG_P)["spec"]
    assert d["embedding"]["vocab_size"] == 160 and d["embedding"]["size"] == 96 and d["head"]["tied"]
    assert d["position"]["kind"] == "none"
    assert d["final_norm"] == {"kind": "rms_norm", "size": 96, "groups": 3, "eps": 1e-5}
    assert [(e["layer"], e["cache"]) for e in d["run_order"]] == [(0, 0), (1, 0), (2, 2), (3, 2), (4, 2)]
    for i, (layer, raw) in enumerate(zip(d["layers"], CONFIG_P["layers"])):
        assert layer["arrangement"] == "parallel"
        m, r = slot(layer, "mixer"), raw["mixer"]
        assert m["kind"] == "latent_attention"
        assert (m["n_head"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]) == (r["heads"], r["dim"], r["rot_dim"], r["vdim"], r["kv_rank"])
        assert m["window"] == r["mask"]["size"] and m["scale"] == r["scale"] and m["rot_base"] == r["rot"]["base"] and m["rot_dims"] == r["rot"]["dims"]
        assert m["own_latent"] == ("kv_from" not in r)
        names = [s["name"] for s in layer["slots"]]
        assert ("feed_forward" in names) == (raw["mlp"] is not None)
        if raw["mlp"] is not None:
            ff = slot(layer, "feed_forward")
            assert ff["inner"] == raw["mlp"]["ff"] and ff["activation"] == "xielu"
        assert slot(layer, "token_input")["dim"] == 8 and slot(layer, "shift")["kind"] == "lerp_previous"
        assert [s["role"] for s in layer["slots"] if s["name"] == "shift"] == ["shift"]
    q = describe_config(CONFIG_Q)["spec"]
    assert all("token_input" not in [s["name"] for s in l["slots"]] for l in q["layers"])
    assert slot(q["layers"][0], "mixer")["window"] == 0 and slot(q["layers"][0], "norm")["groups"] == 1


def test_checkpoint_map_joins_and_slices():
    ck = describe_config(CONFIG_P)["checkpoint"]
    proj = ck["layers.0.mixer.proj.weight"]
    assert [s["name"] for s in proj["sources"]] == ["l0.mix.q", "l0.mix.dkv"] and [s["shape"] for s in proj["sources"]] == [[48, 96], [48, 96]]
    assert [s["name"] for s in ck["layers.1.mixer.proj.weight"]["sources"]] == ["l1.mix.q"]
    assert "layers.1.mixer.latent_norm.weight" not in ck and "layers.0.mixer.latent_norm.weight" in ck
    table = ck["layers.3.token_input.table"]
    assert table["sources"][0] == {"name": "side.embed", "shape": [160, 40]} and table["slice"] == {"axis": 1, "begin": 24, "end": 32}
    assert "layers.2.feed_forward.up.weight" not in ck and ck["layers.4.feed_forward.act"]["sources"][0]["shape"] == [2]


@pytest.mark.parametrize("damage, text", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "latent_attention"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 1), "no latent of its own"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_rank", 48), "differs"),
    (lambda c: c["norm"].__setitem__("groups", 5), "groups"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 5), "rot"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"), "dense"),
])
def test_bad_configurations_are_refused(damage, text):
    c = copy.deepcopy(CONFIG_P)
    damage(c)
    with pytest.raises(LiyabError) as e:
        describe_config(c)
    assert text in str(e.value)


def test_one_row_per_position_and_the_widest_window():
    """A unit of latent rows stores one row per position (not a key and a value), and pages leave a windowed group
    only when the group's window has passed them."""
    need = KvNeed(n_kv_head=1, head_dim=48, window=20, planes=1)
    cache = CacheManager({0: need}, {1 << 20: StateNeed((96,), "float32")}, page_size=16, num_pages=8, max_requests=2)
    assert cache.describe()["bytes_per_token"] == 48 * 4
    assert CacheManager({0: KvNeed(1, 48, 20)}, {}, 16, 8, 2).describe()["bytes_per_token"] == 2 * 48 * 4
    cache.open("a")
    cache.reserve("a", 100)
    cache.commit("a", 100)
    assert cache.pages_in_use()[0] == 2          # positions 81..99 are visible from position 100: pages 5 and 6
    cache.close("a")
    cache.check()
