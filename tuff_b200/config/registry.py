"""One registry from an architecture's name (config.json `architectures[0]`) to
its typed configuration and its model description.

The reference keeps the same map as an enum plus a table of function pointers
(include/tuff_vtable.h:13-58, src/tuff_vtable.c:159-171), keyed by the
architecture string of the model file (src/lfm25_model.c:7-24).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from .base import ConfigError, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict, str], Any]       # raw config.json dict, where -> typed configuration
    model_spec: Callable[[Any], Any]               # typed configuration -> ModelSpec
    config_to_dict: Callable[[Any], dict]          # typed configuration -> config.json dict


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered; known: "
                          f"{', '.join(registered_architectures()) or '(none)'}")
    return _ARCHITECTURES[name]


def config_from_dict(raw: dict, where: str = "config.json"):
    """(architecture, typed configuration) for a config.json dictionary."""
    arch = get_architecture(architecture_name(raw, where))
    return arch, arch.parse_config(raw, where)


def load_config(model_dir: str):
    raw = read_config_json(model_dir)
    return config_from_dict(raw, f"{model_dir}/config.json")


def _register_builtin() -> None:
    from ..models.lfm2 import lfm2_spec
    from .lfm2 import ARCHITECTURE, Lfm2Config
    register_architecture(Architecture(ARCHITECTURE, Lfm2Config.from_dict, lfm2_spec, lambda c: c.to_dict()))


_register_builtin()
