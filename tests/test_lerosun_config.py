"""The Lerosun configuration, its model spec, the tensors it declares and what the cache manager is asked for (pages
for the attention layers, one state row per request for the recurrent ones); no GPU."""
import copy

import pytest
import torch

from helpers import TINY_LEROSUN, make_lerosun_folder
from photon_infer_b200.cache.manager import CacheManager
from photon_infer_b200.config import load_config
from photon_infer_b200.config.lerosun_config import LerosunConfig
from photon_infer_b200.errors import ErrorCode, PhotonError
from photon_infer_b200.models.model import _Skeleton, declared_tensors
from photon_infer_b200.parts.base import PagedCacheSpec, Scaled, StateSpec


def _cfg(name):
    return copy.deepcopy(TINY_LEROSUN[name]["config"])


def load_spec(name_or_dict):
    from photon_infer_b200.config import get_architecture
    arch = get_architecture("Lerosun")
    d = _cfg(name_or_dict) if isinstance(name_or_dict, str) else name_or_dict
    return arch.build_spec(arch.config_class.from_dict(d))


def test_round_trip_and_registry(tmp_path):
    for name in TINY_LEROSUN:
        cfg = LerosunConfig.from_dict(_cfg(name))
        assert LerosunConfig.from_dict(cfg.to_dict()) == cfg
    folder = make_lerosun_folder(str(tmp_path / "m"), "ls_a")
    arch, cfg = load_config(folder)
    assert arch.name == "Lerosun" and cfg.width == 64 and cfg.loop.times == 2
    d = _cfg("ls_b"); d["architectures"] = [d.pop("architecture")]
    assert LerosunConfig.from_dict(d).architecture == "Lerosun"


@pytest.mark.parametrize("path,value,word", [
    (("width",), None, "width"), (("vocab",), 0, "vocab"), (("norm", "eps"), None, "norm.eps"), (("norm",), None, "norm"),
    (("layers", 1, "type"), "conv", "layers[1].type"), (("layers", 0, "mixer", "dim"), None, "dim"),
    (("layers", 0, "mixer", "conv"), None, "conv"), (("layers", 0, "mixer", "conv"), 0, "conv"),
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 1, "mixer", "scale"), "x", "scale"),
    (("layers", 1, "mixer", "vdim"), 48, "vdim"), (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 1, "mixer", "rot", "dims"), 64, "rot.dims"), (("layers", 1, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 0, "mlp", "kind"), "moe", "mlp.kind"), (("layers", 0, "mlp", "ff"), None, "ff"),
    (("loop", "stop"), 9, "loop"), (("loop", "times"), 0, "loop.times"),
])
def test_errors_name_the_key(path, value, word):
    d = _cfg("ls_a")
    node = d
    for k in path[:-1]:
        node = node[k]
    if value is None:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    with pytest.raises(PhotonError) as e:
        LerosunConfig.from_dict(d)
    assert e.value.code == ErrorCode.INVALID_CONFIG and word in str(e.value)


def test_what_the_file_leaves_out_does_not_exist():
    d = _cfg("ls_a")
    m = d["layers"][1]["mixer"]
    for k in ("kv_heads", "vdim", "mask", "rot"):
        m.pop(k)
    d["layers"][0]["mixer"].pop("kv_heads")
    d["loop"] = None
    spec = load_spec(d)
    p = spec.layers[1].mixer.params
    assert p["n_kv_heads"] == p["n_q_heads"] == 4 and p["window"] is None and p["rot_dims"] == 0
    assert spec.layers[0].mixer.params["qk_heads"] == 4
    assert [e.layer for e in spec.run] == [0, 1, 2, 3]


def test_parts_and_their_parameters():
    spec = load_spec("ls_a")
    d, a = spec.layers[0], spec.layers[1]
    assert d.mixer.kind == "delta_rule" and a.mixer.kind == "talking_attention"
    assert d.mixer.params == dict(hidden_size=64, heads=4, qk_heads=2, dim=16, vdim=24, taps=4, eps=1e-5)
    p = a.mixer.params
    assert (p["n_q_heads"], p["n_kv_heads"], p["head_dim"], p["scale"], p["window"], p["rot_dims"], p["rot_base"]) == \
        (4, 2, 32, 0.2, 40, 16, 5000.0)
    assert p["bias"] and p["temperature"] and p["talk"] and p["sink"] and p["output_gate"] and p["values_are_keys"]
    assert a.feed_forward.kind == "gated" and a.feed_forward.params["activation"] == "relu"
    assert a.norm1.kind == "rms_norm" and a.norm1.params["scalar"] and spec.embedding_norm.params["scalar"]
    assert a.scale1.kind == "channel_scale" and a.scale2.params["name"] == "ls2"
    assert spec.layers[2].feed_forward is None and spec.layers[2].scale2 is None and spec.layers[2].norm2 is None
    assert not spec.stream_parts                      # nothing happens between the passes of the looped block


def test_run_list_follows_the_loop():
    run = lambda name: [e.layer for e in load_spec(name).run]
    assert run("ls_a") == [0, 1, 2, 1, 2, 3]
    assert run("ls_b") == [0, 1, 2]
    assert run("ls_c") == [0, 1, 0, 1, 0, 1]
    assert run("ls_d") == [0, 1]
    assert run("ls_e") == [0, 1, 2, 3, 1, 2, 3]
    assert all(e.before is None and e.kv_from is None for e in load_spec("ls_e").run)


def test_declared_tensors():
    d = declared_tensors(load_spec("ls_a"))
    for n in ("embed", "embed.norm", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.ls1", "l0.ls2", "l0.mix.q.conv",
              "l0.mix.k.conv", "l0.mix.v.conv", "l0.mix.A_log", "l0.mix.dt_bias", "l0.mix.a", "l0.mix.b", "l0.mix.norm",
              "l0.mix.g", "l0.mix.o", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down", "l1.mix.q", "l1.mix.q.b", "l1.mix.k.b",
              "l1.mix.talk", "l1.mix.temp", "l1.mix.sink", "l1.mix.g", "l2.ls1"):
        assert n in d, n
    for n in ("l1.mix.v", "l1.mix.q.conv", "l0.mix.q.b", "l0.mix.talk", "l2.norm2", "l2.ls2", "l2.mlp.gate", "loop.step", "l3.mlp.up"):
        assert n not in d, n
    assert d["embed.norm"].shape == () and d["l0.norm1"].shape == () and d["final.norm"].shape == ()
    assert d["l0.ls1"].shape == (64,) and d["l0.mix.q"].shape == (32, 64) and d["l0.mix.v"].shape == (96, 64)
    assert d["l0.mix.q.conv"].shape == (32, 4) and d["l0.mix.v.conv"].shape == (96, 4) and d["l0.mix.a"].shape == (4, 64)
    assert d["l0.mix.norm"].shape == (24,) and d["l0.mix.o"].shape == (64, 96)
    assert d["l1.mix.q"].shape == (128, 64) and d["l1.mix.k"].shape == (64, 64) and d["l1.mix.g"].shape == (4, 64)
    assert d["l1.mix.talk"].shape == (4, 4) and d["l1.mix.o"].shape == (64, 128) and d["l1.mlp.gate"].shape == (80, 64)


def test_cache_needs_and_state():
    sk = _Skeleton(load_spec("ls_a"))
    needs = [(sk.blocks[e.layer].mixer().cache_spec(), sk.blocks[e.layer].mixer().state_spec()) for e in sk.spec.run]
    # a delta layer keeps S [4][16][24] and three projected rows of 2 * 2 * 16 + 4 * 24 channels, no pages
    assert needs[0] == (None, StateSpec((4 * 16 * 24 + 3 * 160,), torch.float32))
    assert needs[1] == (PagedCacheSpec(2, 32, 40), None) and needs[5] == (PagedCacheSpec(1, 64, 24), None)
    assert needs[2][1] == StateSpec((2 * 32 * 16 + 2 * 160,), torch.float32)
    cm = CacheManager(needs, [None] * len(needs), 16, 12, 4, torch.bfloat16, None)
    # the two passes of a looped layer have equal needs: one group of pages, a pool of their own each; and a state each
    assert [g.entries for g in cm.groups] == [[1, 3], [5]]
    assert sorted(cm.states.specs) == [0, 2, 4]
    # a convolution of one tap keeps no rows
    sk = _Skeleton(load_spec("ls_c"))
    assert sk.blocks[1].mixer().state_spec() == StateSpec((72 * 40,), torch.float32)


def test_a_pending_output_with_a_channel_scale():
    from photon_infer_b200.parts.base import delta_pair, delta_terms
    x, s = torch.randn(3, 8).bfloat16(), torch.randn(8)
    d1, d2, sc = delta_terms(Scaled(x, s))
    assert d1 is x and d2 is None and sc is s
    full, none = delta_pair(Scaled(x, s))
    assert none is None and torch.equal(full, x.float() * s)
    assert delta_terms((x, x)) == (x, x, None) and delta_terms(None) == (None, None, None)
