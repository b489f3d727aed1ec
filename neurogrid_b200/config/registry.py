"""One registry from an architecture's name (config.json ``architectures[0]``) to its
typed configuration class.  A configuration class offers ``from_dict(mapping)`` and
``model_spec()``; that is all the rest of the framework asks of an architecture.

The reference keeps a table of model families keyed by name
(``pkg/model/model_config.go:235-295``) and branches on ``ModelType == "lfm2"``
(``pkg/inference/engine_gpu.go:119``); here the table is the only place that names one.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Mapping

from .lfm2 import ConfigError, Lfm2Config

_ARCHITECTURES: Dict[str, Any] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(name: str, config_cls, *, model_type: str | None = None) -> None:
    """Register ``config_cls`` under ``name``; ``model_type`` is an accepted fallback key."""
    _ARCHITECTURES[name] = config_cls
    if model_type:
        _MODEL_TYPES[model_type] = name


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture_name(d: Mapping[str, Any]) -> str:
    archs = d.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        name = archs[0]
    elif d.get("model_type") in _MODEL_TYPES:
        name = _MODEL_TYPES[d["model_type"]]
    else:
        raise ConfigError("config.json names no architecture: give 'architectures': [name]; "
                          f"registered: {', '.join(registered_architectures())}")
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture {name!r}; registered: {', '.join(registered_architectures())}")
    return name


def config_from_dict(d: Mapping[str, Any]):
    return _ARCHITECTURES[architecture_name(d)].from_dict(d)


def load_config(model_dir: str):
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir}")
    with open(path) as f:
        return config_from_dict(json.load(f))


register_architecture("Lfm2ForCausalLM", Lfm2Config, model_type="lfm2")
