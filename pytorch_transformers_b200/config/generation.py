"""Generation options: the reference's names, defaults and meanings for the subset that this
library implements.

``GenerationConfig`` of the reference (src/transformers/generation/configuration_utils.py:98-1329):
defaults :391-493 (``max_length`` 20, ``do_sample`` False, ``temperature`` 1.0, ``top_k`` 50,
``top_p`` 1.0, ``repetition_penalty`` 1.0), validation :585-, loading from
``generation_config.json`` (src/transformers/utils/__init__.py:268) or from the model's
configuration (:1261-1302). Beam search, assisted decoding, constraints and the other
strategies are not part of this library; asking for them is an error, not a silent greedy run.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Dict, Optional, Tuple

GENERATION_CONFIG_NAME = "generation_config.json"
_UNSUPPORTED = {"num_beams": 1, "num_beam_groups": 1, "penalty_alpha": None, "dola_layers": None,
                "typical_p": 1.0, "epsilon_cutoff": 0.0, "eta_cutoff": 0.0, "diversity_penalty": 0.0,
                "encoder_repetition_penalty": 1.0, "no_repeat_ngram_size": 0, "bad_words_ids": None,
                "force_words_ids": None, "constraints": None, "stop_strings": None, "max_time": None,
                "assistant_model": None, "prompt_lookup_num_tokens": None}


@dataclasses.dataclass
class GenerationConfig:
    max_length: int = 20
    max_new_tokens: Optional[int] = None
    min_new_tokens: Optional[int] = None
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int = 50
    top_p: float = 1.0
    min_p: Optional[float] = None
    repetition_penalty: float = 1.0
    num_return_sequences: int = 1
    eos_token_id: Optional[Any] = None
    pad_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    seed: int = 0                      # ours: keys the counter-based sampler (the reference seeds torch globally)
    output_logits: bool = False
    return_dict_in_generate: bool = False

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "GenerationConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        kept = {}
        for k, v in raw.items():
            if k in names:
                if v is not None or k in ("max_new_tokens", "min_new_tokens", "min_p", "eos_token_id",
                                          "pad_token_id", "bos_token_id"):
                    kept[k] = v
            elif k in _UNSUPPORTED and v != _UNSUPPORTED[k] and v is not None:
                raise ValueError(f"generation option {k}={v!r} is not supported by this library "
                                 "(supported strategies: greedy search and sampling)")
        cfg = cls(**kept)
        cfg.validate()
        return cfg

    @classmethod
    def from_pretrained(cls, folder: str, model_config=None) -> "GenerationConfig":
        """``generation_config.json`` if the folder has one, else the token ids of the model's
        configuration (src/transformers/modeling_utils.py:4281-4303)."""
        path = os.path.join(folder, GENERATION_CONFIG_NAME)
        if os.path.isfile(path):
            with open(path, "r", encoding="utf-8") as f:
                raw = json.load(f)
            raw = {k: v for k, v in raw.items() if not k.startswith("_") and k != "transformers_version"}
            return cls.from_dict(raw)
        return cls.from_model_config(model_config)

    @classmethod
    def from_model_config(cls, model_config) -> "GenerationConfig":
        cfg = cls()
        if model_config is not None:
            cfg.eos_token_id = getattr(model_config, "eos_token_id", None)
            cfg.bos_token_id = getattr(model_config, "bos_token_id", None)
            cfg.pad_token_id = getattr(model_config, "pad_token_id", None)
        return cfg

    def updated(self, **kwargs) -> "GenerationConfig":
        """A copy with the given options replaced (generate()'s keyword arguments)."""
        names = {f.name for f in dataclasses.fields(self)}
        for k, v in kwargs.items():
            if k not in names:
                if k in _UNSUPPORTED:
                    if v != _UNSUPPORTED[k] and v is not None:
                        raise ValueError(f"generation option {k}={v!r} is not supported by this library "
                                         "(supported strategies: greedy search and sampling)")
                    continue
                raise ValueError(f"unknown generation option {k!r} (options: {', '.join(sorted(names))})")
        new = dataclasses.replace(self, **{k: v for k, v in kwargs.items() if k in names})
        new.validate()
        return new

    def validate(self) -> None:
        if self.max_new_tokens is not None and self.max_new_tokens <= 0:
            raise ValueError(f"max_new_tokens must be greater than 0, got {self.max_new_tokens}")
        if self.min_new_tokens is not None and self.min_new_tokens < 0:
            raise ValueError(f"min_new_tokens must be >= 0, got {self.min_new_tokens}")
        # logits_process.py:275-283: a strictly positive float
        if not isinstance(self.temperature, (int, float)) or isinstance(self.temperature, bool) or \
                not self.temperature > 0:
            raise ValueError(f"temperature must be a strictly positive float, got {self.temperature!r}")
        if not isinstance(self.top_k, int) or isinstance(self.top_k, bool) or self.top_k < 0:
            raise ValueError(f"top_k must be a non-negative integer (0 switches it off), got {self.top_k!r}")
        if not (0.0 < float(self.top_p) <= 1.0):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p!r}")
        if self.min_p is not None and not (0.0 <= float(self.min_p) <= 1.0):
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p!r}")
        if not float(self.repetition_penalty) > 0:
            raise ValueError(f"repetition_penalty must be strictly positive, got {self.repetition_penalty!r}")
        if self.num_return_sequences < 1:
            raise ValueError("num_return_sequences must be >= 1")
        if self.num_return_sequences > 1 and not self.do_sample:
            raise ValueError("greedy search returns one sequence per prompt: num_return_sequences > 1 needs "
                             "do_sample=True")  # configuration_utils.py validate()

    def eos_ids(self) -> Tuple[int, ...]:
        eos = self.eos_token_id
        if eos is None:
            return ()
        if isinstance(eos, (list, tuple)):
            return tuple(int(e) for e in eos)
        return (int(eos),)

    def new_token_budget(self, longest_prompt: int, max_position_embeddings: Optional[int] = None) -> int:
        """New tokens per sequence, as _prepare_generated_length decides
        (src/transformers/generation/utils.py:1442-1497): ``max_new_tokens`` if set; else a
        non-default ``max_length`` minus the (longest) prompt; else 20 new tokens, the total
        capped by max_position_embeddings."""
        if self.max_new_tokens is not None:
            return int(self.max_new_tokens)
        if self.max_length != 20:
            budget = self.max_length - longest_prompt
        else:
            total = 20 + longest_prompt
            if max_position_embeddings is not None:
                total = min(total, max_position_embeddings)
            budget = total - longest_prompt
        if budget <= 0:
            # utils.py:1409-1415
            raise ValueError(f"the prompt has {longest_prompt} tokens but max_length is {self.max_length}: "
                             "nothing can be generated; raise max_length or set max_new_tokens")
        return budget

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)
