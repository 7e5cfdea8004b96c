"""One registry from an architecture's name to its configuration class and model.

The reference gates architectures with a string list and ``if (a == "...")``
chains (src/model.cpp:55-59, 74-124).  Here ``architectures[0]`` of
``config.json`` is looked up in one table; an unknown name is an error that
lists the registered ones, in the manner of the reference's message at
src/model.cpp:57.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional

from .base import ConfigError, load_config_dict
from .llama import LlamaConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                      # has from_dict(dict) and model_spec()
    build_model: Optional[Callable] = None  # (model_spec, tensors, runtime) -> model; None = the generic decoder


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, build_model: Optional[Callable] = None,
                          replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, build_model)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def lookup_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"architecture '{name}' is not supported (supported: {', '.join(registered_architectures())})") from None


def config_from_dict(d: Dict[str, Any]):
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    arch = lookup_architecture(archs[0])
    return arch, arch.config_class.from_dict(d)


def config_from_model_dir(model_dir: str):
    return config_from_dict(load_config_dict(model_dir))


register_architecture(LlamaConfig.ARCHITECTURE, LlamaConfig)
