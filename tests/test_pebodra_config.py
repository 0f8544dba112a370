"""The Pebodra configuration, its model spec, the tensors it declares and what the cache manager is asked for (pages
for the attention layers that own keys and values, kept for the longest window among their readers; one state row per
request for the recurrent layers); no GPU."""
import copy

import pytest
import torch

from helpers import TINY_PEBODRA, make_pebodra_folder
from photon_infer_b200.cache.manager import CacheManager
from photon_infer_b200.config import load_config
from photon_infer_b200.config.pebodra_config import PebodraConfig
from photon_infer_b200.errors import ErrorCode, PhotonError
from photon_infer_b200.models.model import _Skeleton, declared_tensors
from photon_infer_b200.parts.base import Normed, PagedCacheSpec, StateSpec


def _cfg(name):
    return copy.deepcopy(TINY_PEBODRA[name]["config"])


def load_spec(name_or_dict):
    from photon_infer_b200.config import get_architecture
    arch = get_architecture("Pebodra")
    d = _cfg(name_or_dict) if isinstance(name_or_dict, str) else name_or_dict
    return arch.build_spec(arch.config_class.from_dict(d))


def test_round_trip_and_registry(tmp_path):
    for name in TINY_PEBODRA:
        cfg = PebodraConfig.from_dict(_cfg(name))
        assert PebodraConfig.from_dict(cfg.to_dict()) == cfg
    folder = make_pebodra_folder(str(tmp_path / "m"), "pb_a")
    arch, cfg = load_config(folder)
    assert arch.name == "Pebodra" and cfg.width == 64 and cfg.norm_groups == 2 and cfg.logit_softcap == 20.0
    d = _cfg("pb_b"); d["architectures"] = [d.pop("architecture")]
    assert PebodraConfig.from_dict(d).architecture == "Pebodra"


@pytest.mark.parametrize("path,value,word", [
    (("width",), None, "width"), (("vocab",), 0, "vocab"), (("norm", "eps"), None, "norm.eps"), (("norm",), None, "norm"),
    (("norm", "groups"), 3, "norm.groups"), (("logit_softcap",), -1.0, "logit_softcap"),
    (("layers", 1, "type"), "conv", "layers[1].type"), (("layers", 0, "mixer", "dim"), None, "dim"),
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 0, "mixer", "scale"), "x", "scale"),
    (("layers", 0, "mixer", "diff"), None, "diff"), (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 64, "rot.dims"), (("layers", 0, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 1, "mixer", "gate_cap"), None, "gate_cap"), (("layers", 3, "mixer", "state"), None, "state"),
    (("layers", 3, "mixer", "conv"), 0, "conv"), (("layers", 3, "mixer", "groups"), 3, "groups"),
    (("layers", 3, "mixer", "norm_groups"), 5, "norm_groups"),
    (("layers", 2, "mixer", "kv_from"), 1, "kv_from"), (("layers", 2, "mixer", "kv_from"), 2, "kv_from"),
    (("layers", 2, "mixer", "kv_heads"), 4, "kv_heads"), (("layers", 2, "mixer", "rot", "base"), 10.0, "rot"),
    (("layers", 1, "mlp", "kind"), "glu", "mlp.kind"), (("layers", 1, "mlp", "ff"), None, "ff"),
    (("layers", 0, "mlp", "router", "top"), 9, "router.top"), (("layers", 0, "mlp", "router", "groups", "count"), 4, "router.groups"),
    (("layers", 0, "mlp", "router", "groups", "keep"), 4, "router.groups"), (("layers", 0, "mlp", "expert"), None, "expert"),
])
def test_errors_name_the_key(path, value, word):
    d = _cfg("pb_a")
    node = d
    for k in path[:-1]:
        node = node[k]
    if value is None:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    with pytest.raises(PhotonError) as e:
        PebodraConfig.from_dict(d)
    assert e.value.code == ErrorCode.INVALID_CONFIG and word in str(e.value)


def test_what_the_file_leaves_out_does_not_exist():
    d = _cfg("pb_a")
    d.pop("logit_softcap")
    d["norm"].pop("groups")
    m = d["layers"][0]["mixer"]
    for k in ("kv_heads", "vdim", "mask", "rot"):
        m.pop(k)
    d["layers"][2]["mixer"] = dict(m, kv_from=0)
    d["layers"][0]["mlp"]["router"].pop("groups")
    spec = load_spec(d)
    p = spec.layers[0].mixer.params
    assert p["n_kv_heads"] == p["n_q_heads"] == 4 and p["value_dim"] == 16 and p["window"] is None and p["rot_dims"] == 0
    assert p["cache_window"] is None
    assert spec.logit_softcap is None and spec.final_norm.params["groups"] == 1
    r = spec.layers[0].feed_forward.params
    assert r["groups"] == 1 and r["keep_groups"] is None


def test_parts_and_their_parameters():
    spec = load_spec("pb_a")
    a, mem, reader, ssm = spec.layers
    assert [l.block.kind for l in spec.layers] == ["output_norm"] * 4
    assert (a.mixer.kind, mem.mixer.kind, reader.mixer.kind, ssm.mixer.kind) == \
        ("diff_attention", "matrix_memory", "diff_attention", "state_space")
    p = a.mixer.params
    assert (p["n_q_heads"], p["n_kv_heads"], p["head_dim"], p["value_dim"], p["scale"], p["diff"], p["window"], p["rot_dims"],
            p["rot_base"], p["own_kv"]) == (4, 2, 16, 24, 0.3, 0.2, 40, 8, 5000.0, True)
    assert p["cache_window"] == 56                    # the reader's window is the longer one
    assert reader.mixer.params["own_kv"] is False and reader.mixer.params["window"] == 56
    assert mem.mixer.params == dict(hidden_size=64, heads=2, dim=24, vdim=16, gate_cap=8.0, eps=1e-5)
    assert ssm.mixer.params == dict(hidden_size=64, heads=4, vdim=8, state=16, taps=3, eps=1e-5, groups=2, norm_groups=4)
    assert a.norm1.kind == "group_rms_norm" and a.norm1.params["groups"] == 2 and spec.final_norm.params["groups"] == 2
    f = a.feed_forward.params
    assert a.feed_forward.kind == "moe" and (f["experts"], f["top"], f["expert_size"], f["scoring"], f["groups"], f["keep_groups"],
                                             f["router_bias"], f["gated"]) == (6, 2, 32, "sigmoid", 3, 2, False, True)
    assert mem.feed_forward.kind == "polynorm" and mem.feed_forward.params["intermediate_size"] == 96
    assert reader.feed_forward is None and reader.norm2 is None
    assert spec.logit_softcap == 20.0 and spec.embedding_norm is None and not spec.stream_parts
    assert [(e.layer, e.kv_from) for e in spec.run] == [(0, None), (1, None), (2, 0), (3, None)]
    # two readers, one without a window: everything is kept
    e = load_spec("pb_e")
    assert e.layers[0].mixer.params["cache_window"] is None and e.layers[3].mixer.params["window"] == 8
    assert [x.kv_from for x in e.run] == [None, 0, None, 0, None]


def test_declared_tensors():
    d = declared_tensors(load_spec("pb_a"))
    for n in ("embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.q.b", "l0.mix.k", "l0.mix.k.b", "l0.mix.v",
              "l0.mix.v.b", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.lq1", "l0.mix.lk1", "l0.mix.lq2", "l0.mix.lk2", "l0.mix.o",
              "l0.mix.o.b", "l0.mlp.router", "l0.mlp.e5.gate", "l0.mlp.e0.up", "l0.mlp.e3.down", "l1.mix.i", "l1.mix.i.b",
              "l1.mix.f", "l1.mix.f.b", "l1.mix.g", "l1.mix.norm", "l1.mlp.up", "l1.mlp.down", "l1.mlp.act", "l2.mix.q",
              "l2.mix.q.norm", "l2.mix.lq1", "l2.mix.o.b", "l3.mix.in", "l3.mix.conv", "l3.mix.conv.b", "l3.mix.dt_bias",
              "l3.mix.A_log", "l3.mix.D", "l3.mix.norm", "l3.mix.o"):
        assert n in d, n
    for n in ("l2.mix.k", "l2.mix.k.b", "l2.mix.v", "l2.mix.v.b", "l2.mix.k.norm", "l2.norm2", "l2.mlp.up", "l0.mlp.router.b",
              "l0.mlp.e6.up", "l0.mlp.shared.up", "l1.mlp.gate", "embed.norm", "l3.mlp.e0.gate.b"):
        assert n not in d, n
    assert d["l0.mix.q"].shape == (4 * 2 * 16, 64) and d["l0.mix.k"].shape == (2 * 2 * 16, 64) and d["l0.mix.v"].shape == (48, 64)
    assert d["l0.mix.q.norm"].shape == (16,) and d["l0.mix.lq1"].shape == (16,) and d["l0.mix.o"].shape == (64, 96)
    assert d["l1.mix.q"].shape == (48, 64) and d["l1.mix.v"].shape == (32, 64) and d["l1.mix.i"].shape == (2, 64)
    assert d["l1.mix.norm"].shape == (32,) and d["l1.mlp.act"].shape == (4,)
    assert d["l3.mix.in"].shape == (32 + 32 + 2 * 2 * 16 + 4, 64) and d["l3.mix.conv"].shape == (96, 3) and d["l3.mix.norm"].shape == (32,)


def test_cache_needs_and_state():
    spec = load_spec("pb_a")
    sk = _Skeleton(spec)
    needs = [(sk.blocks[e.layer].mixer().cache_spec() if e.kv_from is None else None, sk.blocks[e.layer].mixer().state_spec())
             for e in spec.run]
    # both maps of a head's key in one cached row; the pages stay for the reader's longer window
    assert needs[0] == (PagedCacheSpec(2, 32, 56, value_dim=24), None) and needs[2] == (None, None)
    # S [2][24][16], n [2][24], m [2]
    assert needs[1] == (None, StateSpec((2 * 24 * 16 + 2 * 24 + 2,), torch.float32))
    # S [4][16][8] and two rows of 32 + 2 * 2 * 16 channels
    assert needs[3] == (None, StateSpec((4 * 16 * 8 + 2 * 96,), torch.float32))
    cm = CacheManager(needs, [e.kv_from for e in spec.run], 16, 12, 4, torch.bfloat16, None)
    assert [g.entries for g in cm.groups] == [[0]] and cm.entry_location[2] == cm.entry_location[0] and cm.entry_shared[2]
    assert sorted(cm.states.specs) == [1, 3]
    # a convolution of one tap keeps no rows
    sk = _Skeleton(load_spec("pb_e"))
    assert sk.blocks[2].mixer().state_spec() == StateSpec((6 * 12 * 4,), torch.float32)


def test_the_window_of_the_cache_is_the_longest_reader_s():
    """Pages behind the owner's own window stay while a reader's longer window still sees them."""
    spec = load_spec("pb_a")
    sk = _Skeleton(spec)
    needs = [(sk.blocks[e.layer].mixer().cache_spec() if e.kv_from is None else None, None) for e in spec.run]
    cm = CacheManager(needs, [e.kv_from for e in spec.run], 8, 40, 2, torch.bfloat16, None)
    cm.add_request("r")
    cm.extend("r", 100)
    cm.commit("r", 100)
    held = [i for i, p in enumerate(cm.groups[0].tables["r"]) if p >= 0]
    assert held[0] == (100 - 56 + 1) // 8 and held[-1] == 99 // 8


def test_a_pending_output_that_waits_for_its_norm():
    from photon_infer_b200.parts.base import delta_pair, delta_terms

    class Doubling:
        def forward(self, x, out_dtype):
            return (2 * x).to(out_dtype)

    x = torch.randn(3, 8).bfloat16()
    full, none = delta_pair(Normed(x, Doubling()))
    assert none is None and full.dtype == torch.float32 and torch.equal(full, 2 * x.float())
    d1, d2, sc = delta_terms(Normed(x, Doubling()))
    assert torch.equal(d1, full) and d2 is None and sc is None
