"""One registry from an architecture's name (``architectures[0]`` of config.json) to
its configuration class and to the function that turns a configuration into a
``ModelSpec`` (the list of layers, their parts and the order they run in).

The reference has one hard-wired model class (include/photon/arch/llama_model.hpp:61)
and no registry; adding an architecture here is one ``register_architecture`` call.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict

from ..errors import ErrorCode, PhotonError
from .model_config import read_config_json


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                       # has from_dict(dict) and to_dict()
    build_spec: Callable[[Any], Any]        # config -> models.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, build_spec: Callable[[Any], Any],
                          replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        known = ", ".join(sorted(_ARCHITECTURES)) or "none"
        raise PhotonError(ErrorCode.UNSUPPORTED_MODEL,
                          f"architecture {name!r} is not registered (known: {known})")
    return _ARCHITECTURES[name]


def registered_architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def architecture_name(d: Dict[str, Any]) -> str:
    """The model class a configuration asks for: ``architectures[0]`` (a list of names) or ``architecture`` (one name)."""
    archs = d.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    if isinstance(d.get("architecture"), str):
        return d["architecture"]
    raise PhotonError(ErrorCode.INVALID_CONFIG,
                      "config.json: key 'architectures' (a non-empty list of names) or 'architecture' (a name) is needed")


def load_config(path: str):
    """Read ``config.json`` and return ``(architecture, typed config)``."""
    d = read_config_json(path)
    arch = get_architecture(architecture_name(d))
    return arch, arch.config_class.from_dict(d)


def _ensure_builtin() -> None:
    # importing the model module registers it
    from ..models import fekopel, finelix, lerosun, llama, pebodra  # noqa: F401
