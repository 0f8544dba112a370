"""Typed configuration of the Lerosun decoder, read from the keys of its ``config.json``.

Nested like the file: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``layers`` (one object per layer:
``type`` names the mixer, ``mixer`` holds its sizes and constants, ``mlp`` its feed-forward or null) and ``loop``
(``start``, ``stop``, ``times``: layers ``start .. stop - 1`` run ``times`` times in a row with the same weights;
absent or null: every layer runs once).  Every size and constant is read here; errors name the key.

Mixers:

* ``attention``: ``heads``, ``kv_heads``, ``dim`` (queries and keys), ``vdim`` (values; the values are the
  projected keys, so it equals ``dim``), ``scale``, optional ``rot`` (``base``, ``dims``: rotation of the first
  ``dims`` numbers of a head) and optional ``mask.size`` (the window; absent: every earlier key is seen);
* ``delta``: ``heads``, ``kv_heads`` (query/key heads), ``dim`` (queries and keys), ``vdim`` (values), ``conv``
  (taps of the short convolutions).

Feed-forward ``kind`` ``dense``: ``ff``.  Optional top-level ``max_positions`` bounds a request's length.
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, Dict, Optional, Tuple

from .nested import bad, num, obj

MIXER_TYPES = ("attention", "delta")
DEFAULT_MAX_POSITIONS = 131072


def _check_mixer(kind: str, m: Any, where: str) -> Dict[str, Any]:
    if not isinstance(m, dict):
        raise bad(f"'{where}' must be an object")
    out: Dict[str, Any] = {"heads": num(m, "heads", where), "dim": num(m, "dim", where)}
    out["kv_heads"] = num(m, "kv_heads", where, default=out["heads"])
    out["vdim"] = num(m, "vdim", where, default=out["dim"])
    if out["heads"] % out["kv_heads"]:
        raise bad(f"'{where}.heads' must be a multiple of '{where}.kv_heads'")
    if kind == "attention":
        out["scale"] = num(m, "scale", where, float)
        if out["vdim"] != out["dim"]:
            raise bad(f"'{where}.vdim' must equal '{where}.dim': the values of this mixer are its projected keys")
        mask = obj(m, "mask", where)
        if mask is not None:
            out["mask"] = {"size": num(mask, "size", where + ".mask")}
        rot = obj(m, "rot", where)
        if rot is not None:
            out["rot"] = {"base": num(rot, "base", where + ".rot", float), "dims": num(rot, "dims", where + ".rot")}
            if out["rot"]["dims"] % 2 or out["rot"]["dims"] > out["dim"]:
                raise bad(f"'{where}.rot.dims' must be even and at most dim")
    else:
        out["conv"] = num(m, "conv", where)
    return out


def _check_mlp(m: Any, where: str) -> Optional[Dict[str, Any]]:
    if m is None:
        return None
    if not isinstance(m, dict):
        raise bad(f"'{where}' must be an object or null")
    if m.get("kind") != "dense":
        raise bad(f"key '{where}.kind' must be 'dense', got {m.get('kind')!r}")
    return {"kind": "dense", "ff": num(m, "ff", where)}


@dataclasses.dataclass(frozen=True)
class LerosunLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclasses.dataclass(frozen=True)
class LerosunLoop:
    start: int
    stop: int
    times: int


@dataclasses.dataclass(frozen=True)
class LerosunConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[LerosunLayer, ...]
    loop: Optional[LerosunLoop]
    max_positions: int = DEFAULT_MAX_POSITIONS

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LerosunConfig":
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
            layers.append(LerosunLayer(l["type"], _check_mixer(l["type"], l.get("mixer"), where + ".mixer"),
                                       _check_mlp(l.get("mlp"), where + ".mlp")))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = LerosunLoop(num(lp, "start", "loop", positive=False, default=0), num(lp, "stop", "loop"),
                               num(lp, "times", "loop"))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise bad(f"'loop' must satisfy 0 <= start < stop <= {len(layers)} layers")
        return cls(architecture=name, vocab=num(d, "vocab", "config"), width=num(d, "width", "config"),
                   norm_eps=num(obj(d, "norm", "config", required=True), "eps", "norm", float), layers=tuple(layers),
                   loop=loop, max_positions=num(d, "max_positions", "config", default=DEFAULT_MAX_POSITIONS))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)} for l in self.layers],
            "loop": dataclasses.asdict(self.loop) if self.loop else None,
        }
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d
