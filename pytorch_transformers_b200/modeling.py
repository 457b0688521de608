"""The Python entry point, in the reference's manner: ``AutoModelForCausalLM.from_pretrained``,
``model.generate``.

``from_pretrained(folder)`` reads config.json, finds the architecture in the registry
(src/transformers/models/auto/auto_factory.py:448-570), builds the model from parts and loads
the safetensors weights (src/transformers/modeling_utils.py:3138-4368 in the reference).
``generate`` takes the reference's arguments where it has them
(src/transformers/generation/utils.py:1908-2401): ``input_ids`` with ``attention_mask``
(left-padded, as the reference wants decoder-only batches, utils.py:2036-2048) or a list of
token lists; ``max_new_tokens``, ``max_length``, ``min_new_tokens``, ``do_sample``,
``temperature``, ``top_k``, ``top_p``, ``min_p``, ``repetition_penalty``,
``num_return_sequences``, ``eos_token_id``, ``pad_token_id``, ``output_logits``,
``return_dict_in_generate``, ``streamer``. Everything runs on one CUDA device through the
library's own kernels.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

import torch

from . import kernels as K
from .cache.paged import PAGE, Cache
from .config.base import ModelConfig
from .config.generation import GenerationConfig
from .config.registry import AutoConfig, lookup, lookup_config, read_raw_config
from .engine.generate import RequestResult, run_generation
from .engine.model import CausalLM
from .sampling.sampler import DeviceSelector
from .weights.loader import load_weights
from .weights.random_init import init_random

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "float": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def resolve_dtype(dtype, config: Optional[ModelConfig] = None, folder: Optional[str] = None) -> torch.dtype:
    """``dtype`` as given, or "auto"/None: the configuration's ``torch_dtype`` if it is one of
    ours, else the dtype that the folder's checkpoint is stored in (32-bit stays 32-bit, 16-bit is
    served in bfloat16), else bfloat16 (the serving precision)."""
    if dtype in (None, "auto"):
        stored = getattr(config, "torch_dtype", None)
        if stored in _DTYPES:
            return _DTYPES[stored]
        if folder is not None:
            from .weights.loader import checkpoint_dtype
            found = checkpoint_dtype(folder)
            if found is not None:
                return found
        return torch.bfloat16
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


@dataclasses.dataclass
class GenerateOutput:
    """``sequences``: prompt + new tokens per request (a padded LongTensor if the input was one);
    ``logits``: per request, float32 [new tokens, vocab] rows the tokens were chosen from."""
    sequences: Any
    logits: Optional[List[torch.Tensor]] = None
    finish_reasons: Optional[List[str]] = None


class _CacheStepper:
    """The generation loop's view of a model and a cache. Prompts that together exceed
    ``max_step_tokens`` are fed in several steps (whole prompts grouped, a longer prompt cut into
    chunks) so that a step's activations stay bounded; the logits of each prompt's last token come
    back in the order asked for, as from one step."""

    def __init__(self, model: CausalLM, cache: Cache, max_step_tokens: int = 16384):
        self.model, self.cache, self.max_step_tokens = model, cache, max(1, int(max_step_tokens))

    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def prepare(self, slots) -> None:
        self.model.prepare_next(self.cache, slots)

    def step_ahead(self, slots, device_tokens):
        return self.model.step_ahead(self.cache, slots, device_tokens)

    def step(self, slots, token_lists):
        total = sum(len(t) for t in token_lists)
        if total <= self.max_step_tokens:
            return self.model.step(self.cache, slots, token_lists, want="last")
        rows = [None] * len(slots)
        group_slots, group_tokens, group_rows, used = [], [], [], 0

        def flush():
            nonlocal group_slots, group_tokens, group_rows, used
            if group_slots:
                out = self.model.step(self.cache, group_slots, group_tokens, want="last")
                for r, i in enumerate(group_rows):
                    if i is not None:
                        rows[i] = out[r]
            group_slots, group_tokens, group_rows, used = [], [], [], 0

        for i, (slot, toks) in enumerate(zip(slots, token_lists)):
            pos = 0
            while pos < len(toks):
                room = self.max_step_tokens - used
                if room == 0:
                    flush()
                    room = self.max_step_tokens
                piece = toks[pos:pos + room]
                pos += len(piece)
                group_slots.append(slot)
                group_tokens.append(piece)
                group_rows.append(i if pos == len(toks) else None)   # only a prompt's end gives its logits
                used += len(piece)
                if pos < len(toks):
                    flush()   # the same slot cannot appear twice in one step
        flush()
        return torch.stack(rows)


class PreTrainedCausalLM(CausalLM):
    """A CausalLM with the loading and generation entry points."""

    generation_config: GenerationConfig

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_pretrained(cls, folder: str, dtype=None, device="cuda", torch_dtype=None,
                        strict: bool = True) -> "PreTrainedCausalLM":
        raw = read_raw_config(folder)
        arch = lookup(raw)
        config = arch.config_cls.from_dict(raw)
        model = cls(arch.spec_builder(config), config, device=device,
                    dtype=resolve_dtype(dtype if dtype is not None else torch_dtype, config, folder))
        load_weights(model, folder, arch.name_rules, strict=strict)
        model.generation_config = GenerationConfig.from_pretrained(folder, config)
        return model

    @classmethod
    def from_config(cls, config: ModelConfig, seed: int = 0, dtype=None, device="cuda") -> "PreTrainedCausalLM":
        """A model with seeded random weights, generated on the device."""
        arch = lookup_config(config)
        model = cls(arch.spec_builder(config), config, device=device, dtype=resolve_dtype(dtype, config))
        init_random(model, seed)
        model.generation_config = GenerationConfig.from_model_config(config)
        return model

    # ------------------------------------------------------------------ generation
    def _ensure_cache(self, max_tokens: int) -> Cache:
        cache = getattr(self, "_cache", None)
        if cache is None or cache.max_tokens < max_tokens or cache.records:
            if cache is not None and cache.records:
                cache = None  # somebody holds sequences in it: leave it alone, use a private one
            self._cache = None
            cache = self.new_cache(max_tokens)
            self._cache = cache
        return cache

    @torch.no_grad()
    def generate(self, inputs=None, generation_config: Optional[GenerationConfig] = None, *, input_ids=None,
                 attention_mask=None, streamer=None, max_batch_size: int = 64, max_step_tokens: int = 16384,
                 on_token: Optional[Callable[[int, int], None]] = None, **kwargs):
        if inputs is None:
            inputs = input_ids
        if inputs is None:
            raise ValueError("generate needs prompts: `inputs`/`input_ids` as a tensor or a list of token lists")
        base = generation_config or getattr(self, "generation_config", None) or GenerationConfig()
        opts = base.updated(**kwargs)
        if opts.eos_token_id is None and "eos_token_id" not in kwargs:
            opts.eos_token_id = getattr(self.config, "eos_token_id", None)

        tensor_in = isinstance(inputs, torch.Tensor)
        if tensor_in:
            ids = inputs.detach().cpu()
            if ids.dim() == 1:
                ids = ids[None]
            if attention_mask is None:
                # inferred from the pad token when it can be told from real tokens (utils.py:579-613)
                pad = opts.pad_token_id
                if pad is not None and (ids == pad).any() and pad not in opts.eos_ids():
                    mask = (ids != pad).long()
                else:
                    mask = torch.ones_like(ids)
            else:
                mask = attention_mask.detach().cpu().long()
            if mask.shape != ids.shape:
                raise ValueError(f"attention_mask {tuple(mask.shape)} does not match input_ids {tuple(ids.shape)}")
            prompts = [ids[b][mask[b].bool()].tolist() for b in range(ids.shape[0])]
            padded_len = ids.shape[1]
        else:
            prompts = [list(map(int, p)) for p in inputs]
            padded_len = max((len(p) for p in prompts), default=0)
        if not prompts:
            raise ValueError("generate got no prompts")

        n_ret = opts.num_return_sequences
        expanded = [p for p in prompts for _ in range(n_ret)]      # utils.py:716-748
        longest = max(len(p) for p in expanded)
        budget = opts.new_token_budget(padded_len if tensor_in else longest,
                                       getattr(self.config, "max_position_embeddings", None))
        max_batch = max(1, min(int(max_batch_size), len(expanded)))
        # the largest batch decides the cache: each request's final length, rounded up to whole pages
        need = 0
        for i in range(0, len(expanded), max_batch):
            need = max(need, sum((len(p) + budget + PAGE - 1) // PAGE * PAGE for p in expanded[i:i + max_batch]))
        cache = self._ensure_cache(need)
        selector = DeviceSelector(self.build.kernels, self.device, self.spec.vocab_size, opts, max_rows=max_batch,
                                  max_history=longest + budget)

        def _on_token(r, tok):
            if on_token is not None:
                on_token(r, tok)

        # The reference pushes the prompts and then every step's tokens to the streamer, a row per request
        # (streamers.py:27-233; utils.py:3287-3299; rows that have ended get the pad token). That is done
        # here when the requests run as one batch; several batches run one after another, and then every
        # finished request is handed over once at the end.
        stream_steps = streamer is not None and len(expanded) <= max_batch
        pad_stream = opts.pad_token_id if opts.pad_token_id is not None else (opts.eos_ids() or [0])[0]
        if stream_steps:
            if tensor_in:
                streamer.put(ids.repeat_interleave(n_ret, 0) if n_ret > 1 else ids)
            else:
                first = torch.full((len(expanded), longest), int(pad_stream), dtype=torch.long)
                for i, pr in enumerate(expanded):                  # left-padded, as the reference wants batches
                    first[i, longest - len(pr):] = torch.tensor(pr, dtype=torch.long)
                streamer.put(first)

        def _on_step(step_tokens):
            streamer.put(torch.tensor([step_tokens.get(i, int(pad_stream)) for i in range(len(expanded))],
                                      dtype=torch.long))

        results = run_generation(_CacheStepper(self, cache, max_step_tokens), selector, expanded, opts, budget, max_batch,
                                 on_token=_on_token if on_token is not None else None,
                                 keep_logits=opts.output_logits, on_step=_on_step if stream_steps else None)
        self.check_errors()
        if streamer is not None:
            if not stream_steps:
                for res in results:
                    streamer.put(torch.tensor(res.prompt + res.tokens))
            streamer.end()

        if tensor_in:
            pad = opts.pad_token_id
            if pad is None:
                eos = opts.eos_ids()
                pad = eos[0] if eos else 0                         # utils.py:1864-1872
            width = padded_len + max(len(r.tokens) for r in results)
            seqs = torch.full((len(results), width), int(pad), dtype=torch.long)
            for i, res in enumerate(results):
                src = ids[i // n_ret]
                seqs[i, :padded_len] = src
                seqs[i, padded_len:padded_len + len(res.tokens)] = torch.tensor(res.tokens, dtype=torch.long)
            sequences: Any = seqs.to(inputs.device)
        else:
            sequences = [res.prompt + res.tokens for res in results]
        if opts.return_dict_in_generate or opts.output_logits:
            logits = [torch.stack(r.logits) for r in results] if opts.output_logits else None
            return GenerateOutput(sequences, logits, [r.finish_reason for r in results])
        return sequences


class AutoModelForCausalLM:
    """``AutoModelForCausalLM.from_pretrained(folder)``: the model class is chosen by config.json."""

    @staticmethod
    def from_pretrained(folder: str, dtype=None, device="cuda", torch_dtype=None,
                        strict: bool = True) -> PreTrainedCausalLM:
        return PreTrainedCausalLM.from_pretrained(folder, dtype=dtype, device=device, torch_dtype=torch_dtype,
                                                  strict=strict)

    @staticmethod
    def from_config(config: ModelConfig, seed: int = 0, dtype=None, device="cuda") -> PreTrainedCausalLM:
        return PreTrainedCausalLM.from_config(config, seed=seed, dtype=dtype, device=device)


class FalconForCausalLM(PreTrainedCausalLM):
    """Falcon by name. The class adds nothing: the architecture lives in models/falcon.py as data."""

    @classmethod
    def from_pretrained(cls, folder: str, dtype=None, device="cuda", torch_dtype=None, strict: bool = True):
        raw = read_raw_config(folder)
        if lookup(raw).model_type != "falcon":
            raise ValueError(f"{folder!r} holds a {raw.get('model_type')!r} model, not a Falcon")
        return super().from_pretrained(folder, dtype=dtype, device=device, torch_dtype=torch_dtype, strict=strict)
