"""Random-weights mode: fill a model from a seed, or write a model folder
(config.json + model.safetensors) from a configuration and a seed.

Law: matrices and bias vectors N(0, std) with the parameter's declared std (0.02 unless the
part says otherwise), norm gains 1 + N(0, std). A value depends on (seed, tensor name, element
index) alone (weights/generator.py), so it depends neither on the order of generation nor on
which other tensors exist, and it is the same whether the host computes it or the device
(csrc/fill_normal.cu). The storage dtype is part of the law: a bfloat16 model holds the values
rounded to bfloat16, in the file and on the device, so ``from_config(config, seed)`` and
``write_random_model(config, seed)`` followed by ``from_pretrained`` are the same model. The
reference initialises N(0, initializer_range) with zero biases and unit gains from torch's
global generator (src/transformers/models/falcon/modeling_falcon.py:794-808); gains and biases
are randomised here so that tests notice a norm or a bias that is skipped.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import generator
from .safetensors_io import SAFE_WEIGHTS_NAME, write_safetensors

_LAWS = {"normal": 0.0, "one_plus_normal": 1.0}


def random_tensor(name: str, decl, seed: int, device, dtype: torch.dtype,
                  store_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """The tensor ``name`` under ``seed`` as ``dtype`` on ``device``, holding the values that a file
    of ``store_dtype`` (default: ``dtype``) holds. On a CUDA device the fill kernel writes the
    tensor in place (no float32 staging copy); elsewhere the host generator does."""
    device = torch.device(device)
    if decl.role == "int" or decl.init == "zeros":
        return torch.zeros(decl.shape, dtype=torch.int32 if decl.role == "int" else dtype, device=device)
    if decl.init not in _LAWS:
        raise ValueError(f"unknown init law {decl.init!r} for {name}")
    offset = _LAWS[decl.init]
    store_dtype = store_dtype or dtype
    as_bf16 = store_dtype == torch.bfloat16
    if device.type == "cuda":
        from .. import kernels
        out = torch.empty(decl.shape, dtype=dtype, device=device)
        kernels.fill_normal(out, generator.tensor_key(seed, name), decl.std, offset,
                            round_bf16=as_bf16 and dtype == torch.float32)
        return out
    n = 1
    for s in decl.shape:
        n *= int(s)
    values = generator.normal_values(seed, name, 0, n, decl.std, offset, bf16=as_bf16)
    return torch.from_numpy(values).reshape(decl.shape).to(dtype)


def init_random(model, seed: int) -> None:
    """Fill ``model`` with seeded random weights, generated on its device."""
    tensors = {}
    for name, (part, logical, decl) in model.param_table().items():
        tensors[name] = random_tensor(name, decl, seed, model.device, model.device_dtype(decl), model.dtype)
    model.bind(tensors)


def write_random_model(config, seed: int, folder: str, dtype: torch.dtype = torch.bfloat16,
                       device: Optional[str] = None) -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors`` for ``config`` with weights
    drawn from ``seed``. All tensors are stored in ``dtype``. Tensors are generated one at a time
    (on ``device`` if given, else on the host; the bits are the same), so large models stream to
    disk."""
    from ..config.registry import lookup_config
    from ..engine.model import CausalLM

    arch = lookup_config(config)
    spec = arch.spec_builder(config)
    gen_device = torch.device(device or "cpu")
    # a model skeleton without weights: parts are built only to declare their parameters
    skeleton = CausalLM(spec, config, device="cpu", dtype=dtype)
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
