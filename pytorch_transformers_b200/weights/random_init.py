"""Random-weights mode: fill a model from a seed, or write a model folder
(config.json + model.safetensors) from a configuration and a seed.

Law: matrices and bias vectors N(0, std) with the parameter's declared std (0.02 unless the
part says otherwise), norm gains 1 + N(0, std). Every tensor has its own generator, seeded
from (seed, tensor name), so a tensor's values depend neither on the order of generation nor on
which other tensors exist. The reference initialises N(0, initializer_range) with zero biases
and unit gains (src/transformers/models/falcon/modeling_falcon.py:794-808); gains and biases
are randomised here so that tests notice a norm or a bias that is skipped.
"""
from __future__ import annotations

import hashlib
import os
from typing import Optional

import torch

from .safetensors_io import SAFE_WEIGHTS_NAME, write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & (2 ** 63 - 1)


def random_tensor(name: str, decl, seed: int, device, dtype: torch.dtype) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    if decl.role == "int":
        return torch.zeros(decl.shape, dtype=torch.int32, device=device)
    t = torch.empty(decl.shape, dtype=torch.float32, device=device)
    # large matrices are filled in slices to bound the float32 staging memory
    t.normal_(0.0, decl.std, generator=gen)
    if decl.init == "one_plus_normal":
        t += 1.0
    elif decl.init == "zeros":
        t.zero_()
    elif decl.init != "normal":
        raise ValueError(f"unknown init law {decl.init!r} for {name}")
    return t.to(dtype)


def init_random(model, seed: int) -> None:
    """Fill ``model`` with seeded random weights, generated on its device."""
    tensors = {}
    for name, (part, logical, decl) in model.param_table().items():
        tensors[name] = random_tensor(name, decl, seed, model.device, model.device_dtype(decl))
    model.bind(tensors)


def write_random_model(config, seed: int, folder: str, dtype: torch.dtype = torch.bfloat16,
                       device: Optional[str] = None) -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors`` for ``config`` with weights
    drawn from ``seed``. All tensors are stored in ``dtype``. Tensors are generated one at a time
    (on ``device`` if given, else on the host), so large models stream to disk."""
    from ..config.registry import lookup_config
    from ..engine.model import CausalLM

    arch = lookup_config(config)
    spec = arch.spec_builder(config)
    gen_device = torch.device(device or "cpu")
    # a model skeleton without weights: parts are built only to declare their parameters
    skeleton = CausalLM(spec, config, device=gen_device, dtype=dtype)
    table = skeleton.param_table()
    plan = [(name, dtype, tuple(decl.shape)) if decl.role != "int" else (name, torch.int32, tuple(decl.shape))
            for name, (_, _, decl) in table.items()]

    def produce():
        for name, (_, _, decl) in table.items():
            want = torch.int32 if decl.role == "int" else dtype
            yield name, random_tensor(name, decl, seed, gen_device, want).cpu()

    os.makedirs(folder, exist_ok=True)
    config.save_pretrained(folder)
    write_safetensors(os.path.join(folder, SAFE_WEIGHTS_NAME), produce(), metadata={"format": "pt"}, plan=plan)
    return folder
