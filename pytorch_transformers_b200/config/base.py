"""Typed configuration base: a dataclass filled from an architecture's own config.json keys.

Plays the role of ``PretrainedConfig`` (src/transformers/configuration_utils.py:51) for a
library that only reads local model folders: ``from_dict`` (configuration_utils.py:714-772),
``to_dict`` (:866), unknown keys kept (:318-324), and the common fields every decoder
carries (``tie_word_embeddings`` default true :221-223, ``architectures`` :239,
``bos/pad/eos_token_id`` :268-271, ``torch_dtype`` :217).
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, ClassVar, Dict, Optional, Tuple

from ..utils import logging as log

CONFIG_NAME = "config.json"  # src/transformers/utils/__init__.py:263
_logger = log.get_logger(__name__)


class ConfigError(ValueError):
    """A config.json value (or combination of values) that the library cannot build."""


@dataclasses.dataclass
class ModelConfig:
    """Fields shared by every architecture. Subclasses add their own typed fields.

    ``aliases`` maps an old key to its field name; ``model_type`` is the registry key.
    Keys that no field claims are kept in ``extra`` and written back by ``to_dict``.
    """

    model_type: ClassVar[str] = ""
    aliases: ClassVar[Dict[str, str]] = {}

    architectures: Optional[Tuple[str, ...]] = None
    tie_word_embeddings: bool = True
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[Any] = None  # int or list of ints
    pad_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    extra: Dict[str, Any] = dataclasses.field(default_factory=dict)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        raw = dict(raw)
        raw.pop("model_type", None)
        names = {f.name for f in dataclasses.fields(cls)} - {"extra"}
        kwargs: Dict[str, Any] = {}
        extra: Dict[str, Any] = {}
        # aliases first, so that an explicit new-style key wins over an old one
        for old, new in cls.aliases.items():
            if old in raw:
                value = raw.pop(old)
                if new not in raw:
                    raw[new] = value
        for key, value in raw.items():
            if key in names:
                kwargs[key] = value
            else:
                extra[key] = value
        if isinstance(kwargs.get("architectures"), list):
            kwargs["architectures"] = tuple(kwargs["architectures"])
        cfg = cls(**kwargs)
        cfg.extra = extra
        if extra:
            _logger.debug("%s keeps config keys that it has no field for: %s", cls.__name__, ", ".join(sorted(extra)))
        return cfg

    @classmethod
    def from_json_file(cls, path: str) -> "ModelConfig":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    @classmethod
    def from_pretrained(cls, folder: str) -> "ModelConfig":
        path = os.path.join(folder, CONFIG_NAME)
        if not os.path.isfile(path):
            raise FileNotFoundError(f"no {CONFIG_NAME} in model folder {folder!r}")
        return cls.from_json_file(path)

    # ------------------------------------------------------------------ output
    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"model_type": self.model_type}
        for f in dataclasses.fields(self):
            if f.name == "extra":
                continue
            value = getattr(self, f.name)
            if isinstance(value, tuple):
                value = list(value)
            out[f.name] = value
        for key, value in self.extra.items():
            out.setdefault(key, value)
        return out

    def save_pretrained(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, CONFIG_NAME), "w", encoding="utf-8") as f:
            json.dump(self.to_dict(), f, indent=2, sort_keys=True)
            f.write("\n")

    # ------------------------------------------------------------------ helpers
    def eos_token_ids(self) -> Tuple[int, ...]:
        """The stop set: ``eos_token_id`` may be an int or a list (generation/utils.py:1859-1861)."""
        eos = self.eos_token_id
        if eos is None:
            return ()
        if isinstance(eos, (list, tuple)):
            return tuple(int(e) for e in eos)
        return (int(eos),)


def _require(cond: bool, message: str) -> None:
    if not cond:
        raise ConfigError(message)
