"""One registry from an architecture's name to its configuration class and model builder.

Lookup goes by config.json's ``model_type`` first and by its ``architectures`` second, as
``AutoConfig`` / ``AutoModelForCausalLM`` do
(src/transformers/models/auto/configuration_auto.py:1073-1088, auto_factory.py:387-400); an
unknown name is a ValueError that lists what is registered (configuration_auto.py:1095-1099).
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Callable, Dict, Optional, Tuple

from .base import CONFIG_NAME, ModelConfig


@dataclasses.dataclass
class Architecture:
    model_type: str
    architectures: Tuple[str, ...]
    config_cls: type
    spec_builder: Callable[[Any], Any]          # config -> parts.ModelSpec
    name_rules: Dict[str, Any] = dataclasses.field(default_factory=dict)


_BY_TYPE: Dict[str, Architecture] = {}
_BY_CLASS: Dict[str, Architecture] = {}


def register_architecture(model_type: str, architectures, config_cls: type, spec_builder, name_rules=None,
                          aliases=()) -> Architecture:
    arch = Architecture(model_type, tuple(architectures), config_cls, spec_builder, dict(name_rules or {}))
    _BY_TYPE[model_type] = arch
    for a in aliases:
        _BY_TYPE[a] = arch
    for a in arch.architectures:
        _BY_CLASS[a] = arch
    return arch


def registered() -> Dict[str, Architecture]:
    return dict(_BY_TYPE)


def lookup(raw_config: Dict[str, Any]) -> Architecture:
    mt = raw_config.get("model_type")
    if mt in _BY_TYPE:
        return _BY_TYPE[mt]
    for a in raw_config.get("architectures") or ():
        if a in _BY_CLASS:
            return _BY_CLASS[a]
    raise ValueError(f"unrecognised model: model_type={mt!r}, architectures={raw_config.get('architectures')!r}. "
                     f"Registered model types: {', '.join(sorted(_BY_TYPE)) or 'none'}; architectures: "
                     f"{', '.join(sorted(_BY_CLASS)) or 'none'}")


def lookup_config(config: ModelConfig) -> Architecture:
    for arch in _BY_TYPE.values():
        if type(config) is arch.config_cls:
            return arch
    raise ValueError(f"no architecture is registered for configuration class {type(config).__name__} "
                     f"(registered: {', '.join(sorted(_BY_TYPE)) or 'none'})")


def read_raw_config(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, CONFIG_NAME)
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no {CONFIG_NAME} in model folder {folder!r}")
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


class AutoConfig:
    """``AutoConfig.from_pretrained(folder)`` -> the typed configuration of the folder's model."""

    @staticmethod
    def from_pretrained(folder: str) -> ModelConfig:
        raw = read_raw_config(folder)
        return lookup(raw).config_cls.from_dict(raw)

    @staticmethod
    def for_model(model_type: str, **kwargs) -> ModelConfig:
        return lookup({"model_type": model_type}).config_cls.from_dict(kwargs)
