"""One registry from an architecture's name to its configuration class.

A configuration class has `from_dict(config.json as a dict)`, `to_dict()` and `to_spec()`
(a `ModelSpec`).  The name is `architectures[0]` of config.json, or is found from
`model_type`; if both are present they must agree, and an unknown name is refused with the
list of what is served (x0ne-infer/src/arch.rs:56-142).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Mapping, Tuple

from .spec import ConfigError, ModelSpec

_BY_NAME: Dict[str, Any] = {}
_BY_MODEL_TYPE: Dict[str, str] = {}


def register_architecture(name: str, model_type: str, config_class: Any) -> None:
    """Adds an architecture; naming one twice is an error (a silent override hides a typo)."""
    if name in _BY_NAME:
        raise ValueError(f"architecture {name!r} is already registered")
    if model_type in _BY_MODEL_TYPE:
        raise ValueError(f"model_type {model_type!r} is already registered")
    _BY_NAME[name] = config_class
    _BY_MODEL_TYPE[model_type] = name


def unregister_architecture(name: str) -> None:
    cls = _BY_NAME.pop(name, None)
    if cls is not None:
        for mt, n in list(_BY_MODEL_TYPE.items()):
            if n == name:
                del _BY_MODEL_TYPE[mt]


def architectures() -> Tuple[str, ...]:
    return tuple(sorted(_BY_NAME))


def detect(config: Mapping[str, Any]) -> str:
    """The registered architecture a config.json names."""
    archs = config.get("architectures")
    mt = config.get("model_type")
    by_class = None
    if archs is not None:
        if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
            raise ConfigError(f"config.json: architectures must name exactly one class, got {archs!r}")
        by_class = archs[0]
        if by_class not in _BY_NAME:
            raise ConfigError(f"config.json: architecture {by_class!r} is not served; "
                              f"served: {', '.join(architectures())}")
    by_type = None
    if mt is not None:
        if mt not in _BY_MODEL_TYPE:
            raise ConfigError(f"config.json: model_type {mt!r} is not served; "
                              f"served: {', '.join(sorted(_BY_MODEL_TYPE))}")
        by_type = _BY_MODEL_TYPE[mt]
    if by_class is None and by_type is None:
        raise ConfigError("config.json: neither architectures nor model_type is given")
    if by_class is not None and by_type is not None and by_class != by_type:
        raise ConfigError(f"config.json: architectures names {by_class!r} but model_type "
                          f"{mt!r} is {by_type!r}")
    return by_class or by_type


def config_from_dict(config: Mapping[str, Any]):
    return _BY_NAME[detect(config)].from_dict(config)


def config_from_folder(folder: str):
    path = os.path.join(folder, "config.json")
    try:
        with open(path) as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"config.json: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError("config.json: not a JSON object")
    return config_from_dict(d)


def spec_from_folder(folder: str) -> ModelSpec:
    return config_from_folder(folder).to_spec()
