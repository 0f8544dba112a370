"""Typed configuration of the Pebodra decoder, read from the keys of its ``config.json``.

Nested like the file: ``architecture``, ``vocab``, ``width``, ``norm`` (``eps``, ``groups``: the parts of the grouped RMS
norms on the sublayers' outputs and at the end), optional ``logit_softcap``, and ``layers`` (one object per layer:
``type`` names the mixer, ``mixer`` holds its sizes and constants, ``mlp`` its feed-forward or null).  Every size and
constant is read here; errors name the key.  What the file leaves out does not exist (no window, no rotation, no
router groups, no bound on the logits).

Mixers:

* ``attention`` (two score maps per head): ``heads``, ``kv_heads``, ``dim`` (queries and keys, per map), ``vdim`` (values),
  ``scale``, ``diff``, optional ``rot`` (``base``, ``dims``: rotation of the first ``dims`` numbers of a map), optional
  ``mask.size`` (the window), optional ``kv_from`` (an earlier attention layer whose keys and values this one reads);
* ``mamba2``: ``heads``, ``vdim``, ``state``, ``groups``, ``conv`` (taps of the short convolution), ``norm_groups``;
* ``mlstm``: ``heads``, ``dim``, ``vdim``, ``gate_cap``.

Feed-forward ``kind`` ``dense``: ``ff``.  ``kind`` ``moe``: ``expert.ff``, ``router.experts``, ``router.top`` and optional
``router.groups`` (``count``, ``keep``).  Optional top-level ``max_positions`` bounds a request's length.
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, Dict, Optional, Tuple

from .nested import bad, num, obj

MIXER_TYPES = ("attention", "mamba2", "mlstm")
DEFAULT_MAX_POSITIONS = 131072


def _check_mixer(kind: str, m: Any, where: str, index: int, before) -> Dict[str, Any]:
    if not isinstance(m, dict):
        raise bad(f"'{where}' must be an object")
    out: Dict[str, Any] = {"heads": num(m, "heads", where)}
    if kind == "attention":
        out["kv_heads"] = num(m, "kv_heads", where, default=out["heads"])
        out["dim"] = num(m, "dim", where)
        out["vdim"] = num(m, "vdim", where, default=out["dim"])
        if out["heads"] % out["kv_heads"]:
            raise bad(f"'{where}.heads' must be a multiple of '{where}.kv_heads'")
        out["scale"] = num(m, "scale", where, float)
        out["diff"] = num(m, "diff", where, float, positive=False)
        mask = obj(m, "mask", where)
        if mask is not None:
            out["mask"] = {"size": num(mask, "size", where + ".mask")}
        rot = obj(m, "rot", where)
        if rot is not None:
            out["rot"] = {"base": num(rot, "base", where + ".rot", float), "dims": num(rot, "dims", where + ".rot")}
            if out["rot"]["dims"] % 2 or out["rot"]["dims"] > out["dim"]:
                raise bad(f"'{where}.rot.dims' must be even and at most dim")
        if m.get("kv_from") is not None:
            src = num(m, "kv_from", where, positive=False)
            if not 0 <= src < index or before[src].type != "attention" or "kv_from" in before[src].mixer:
                raise bad(f"'{where}.kv_from' must name an earlier attention layer that has keys and values of its own")
            theirs = before[src].mixer
            for key in ("kv_heads", "dim", "vdim"):
                if theirs[key] != out[key]:
                    raise bad(f"'{where}.{key}' must equal that of layer {src}, whose keys and values it reads")
            if theirs.get("rot") != out.get("rot"):
                raise bad(f"'{where}.rot' must equal that of layer {src}, whose keys it reads")
            out["kv_from"] = src
    elif kind == "mamba2":
        out["vdim"] = num(m, "vdim", where)
        out["state"] = num(m, "state", where)
        out["groups"] = num(m, "groups", where, default=1)
        out["conv"] = num(m, "conv", where)
        out["norm_groups"] = num(m, "norm_groups", where, default=1)
        if out["heads"] % out["groups"]:
            raise bad(f"'{where}.heads' must be a multiple of '{where}.groups'")
        if (out["heads"] * out["vdim"]) % out["norm_groups"]:
            raise bad(f"'{where}.norm_groups' must divide heads * vdim")
    else:
        out["dim"] = num(m, "dim", where)
        out["vdim"] = num(m, "vdim", where, default=out["dim"])
        out["gate_cap"] = num(m, "gate_cap", where, float)
    return out


def _check_mlp(m: Any, where: str) -> Optional[Dict[str, Any]]:
    if m is None:
        return None
    if not isinstance(m, dict):
        raise bad(f"'{where}' must be an object or null")
    kind = m.get("kind")
    if kind == "dense":
        return {"kind": "dense", "ff": num(m, "ff", where)}
    if kind != "moe":
        raise bad(f"key '{where}.kind' must be 'dense' or 'moe', got {kind!r}")
    r = obj(m, "router", where, required=True)
    router: Dict[str, Any] = {"experts": num(r, "experts", where + ".router"), "top": num(r, "top", where + ".router")}
    if router["top"] > router["experts"]:
        raise bad(f"'{where}.router.top' cannot exceed the number of experts")
    g = obj(r, "groups", where + ".router")
    if g is not None:
        router["groups"] = {"count": num(g, "count", where + ".router.groups"), "keep": num(g, "keep", where + ".router.groups")}
        count, keep = router["groups"]["count"], router["groups"]["keep"]
        if router["experts"] % count or keep > count or keep * (router["experts"] // count) < router["top"]:
            raise bad(f"'{where}.router.groups': the experts must split into equal groups, and the kept groups must hold "
                      "at least 'top' experts")
    return {"kind": "moe", "expert": {"ff": num(obj(m, "expert", where, required=True), "ff", where + ".expert")}, "router": router}


@dataclasses.dataclass(frozen=True)
class PebodraLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclasses.dataclass(frozen=True)
class PebodraConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    layers: Tuple[PebodraLayer, ...]
    logit_softcap: Optional[float] = None
    max_positions: int = DEFAULT_MAX_POSITIONS

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PebodraConfig":
        name = d.get("architecture")
        if not isinstance(name, str):
            archs = d.get("architectures")
            if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
                raise bad("key 'architecture' must name the model class")
            name = archs[0]
        layers_in = d.get("layers")
        if not isinstance(layers_in, list) or not layers_in:
            raise bad("key 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(layers_in):
            where = f"layers[{i}]"
            if not isinstance(l, dict) or l.get("type") not in MIXER_TYPES:
                raise bad(f"'{where}.type' must be one of {', '.join(MIXER_TYPES)}")
            layers.append(PebodraLayer(l["type"], _check_mixer(l["type"], l.get("mixer"), where + ".mixer", i, layers),
                                       _check_mlp(l.get("mlp"), where + ".mlp")))
        norm = obj(d, "norm", "config", required=True)
        width = num(d, "width", "config")
        groups = num(norm, "groups", "norm", default=1)
        if width % groups:
            raise bad("'norm.groups' must divide 'width'")
        cap = d.get("logit_softcap")
        return cls(architecture=name, vocab=num(d, "vocab", "config"), width=width, norm_eps=num(norm, "eps", "norm", float),
                   norm_groups=groups, layers=tuple(layers),
                   logit_softcap=num(d, "logit_softcap", "config", float) if cap is not None else None,
                   max_positions=num(d, "max_positions", "config", default=DEFAULT_MAX_POSITIONS))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
            "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)} for l in self.layers],
        }
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d
