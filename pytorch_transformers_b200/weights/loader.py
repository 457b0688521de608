"""Weights from safetensors by tensor name, with one error that says everything that is wrong.

The model's parts declare their parameters and the architecture's spec gives each a checkpoint
name (engine.model.CausalLM.param_table). Loading matches that table against the archive(s):
missing tensors, tensors nobody asked for and tensors of the wrong shape are collected and
raised together as one ``WeightError``. The reference only warns about missing and unexpected
keys and leaves missing tensors at their random initialisation
(src/transformers/modeling_utils.py:4893-4912) and raises on shape mismatches (:4884-4891);
here all three are errors.

Precision on the device: matrices are kept in the model dtype (bfloat16 for serving),
gain and bias vectors in float32 (lossless for any stored dtype), integer tables as int32.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..utils import logging as log
from .safetensors_io import open_checkpoint

_logger = log.get_logger(__name__)

_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)


class WeightError(RuntimeError):
    """The checkpoint does not fit the model. ``missing``, ``unexpected`` and ``mismatched``
    hold the details that the message lists."""

    def __init__(self, folder: str, missing: List[str], unexpected: List[str], mismatched: List[str]):
        self.missing, self.unexpected, self.mismatched = missing, unexpected, mismatched
        lines = [f"the weights in {folder!r} do not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if mismatched:
            lines.append(f"  wrong shape or dtype ({len(mismatched)}): " + "; ".join(mismatched))
        super().__init__("\n".join(lines))


def checkpoint_dtype(folder: str) -> Optional[torch.dtype]:
    """The dtype that the folder's archives store their matrices in: float32 if the first floating-point
    tensor of two or more dimensions is stored in 32-bit, bfloat16 if it is stored in 16 bits (bfloat16 or
    float16, which is converted at load), None if there is no such tensor. It is what ``dtype="auto"``
    means when config.json names no ``torch_dtype`` (the reference looks at the first floating-point tensor
    of the state dict too, src/transformers/modeling_utils.py:4037-4046)."""
    files, where = open_checkpoint(folder)
    try:
        for name, f in where.items():
            e = f.entries[name]
            if e.dtype in _FLOATS and len(e.shape) >= 2:
                return torch.float32 if e.dtype in (torch.float32, torch.float64) else torch.bfloat16
        return None
    finally:
        for f in files:
            f.close()


def load_weights(model, folder: str, name_rules: Optional[dict] = None, strict: bool = True) -> None:
    """Read every parameter of ``model`` from the archive(s) in ``folder`` and bind them. With
    ``strict=False`` tensors that the model does not ask for are reported as a warning instead of an
    error (missing tensors and wrong shapes stay errors: the model could not run)."""
    rules = name_rules or {}
    prefix = rules.get("optional_prefix")
    ignore = tuple(rules.get("ignore_suffixes", ()))
    table = model.param_table()
    files, where = open_checkpoint(folder)
    try:
        # canonical name -> (file, name in the file)
        stored = {n: (f, n) for n, f in where.items() if not (ignore and n.endswith(ignore))}
        # a checkpoint saved from the bare decoder lacks the prefix that the full model's names carry
        if prefix and stored and not any(n.startswith(prefix) for n in stored):
            stored = {(prefix + n if prefix + n in table else n): fn for n, fn in stored.items()}
        tied_head = model.spec.head_name is None
        missing = [n for n in table if n not in stored]
        unexpected = [n for n in stored if n not in table]
        if tied_head:
            # a tied head may still be stored; it must then be the embedding itself
            unexpected = [n for n in unexpected if n != "lm_head.weight"]
        mismatched: List[str] = []
        for name, (part, logical, decl) in table.items():
            if name not in stored:
                continue
            f, real = stored[name]
            e = f.entries[real]
            if tuple(e.shape) != tuple(decl.shape):
                mismatched.append(f"{name}: stored {list(e.shape)}, model wants {list(decl.shape)}")
            elif decl.role == "int" and e.dtype.is_floating_point:
                mismatched.append(f"{name}: stored as {e.dtype}, model wants an integer table")
            elif decl.role != "int" and e.dtype not in _FLOATS:
                mismatched.append(f"{name}: stored as {e.dtype}, model wants floating point")
        if unexpected and not strict and not missing and not mismatched:
            _logger.warning("%s: %d tensors are not used by the model: %s", folder, len(unexpected),
                            ", ".join(sorted(unexpected)))
            unexpected = []
        if missing or unexpected or mismatched:
            raise WeightError(folder, sorted(missing), sorted(unexpected), mismatched)
        tensors: Dict[str, torch.Tensor] = {}
        for name, (part, logical, decl) in table.items():
            f, real = stored[name]
            host = f.tensor(real)
            tensors[name] = host.to(device=model.device, dtype=model.device_dtype(decl))
        if tied_head and "lm_head.weight" in stored:
            f, real = stored["lm_head.weight"]
            head = f.tensor(real)
            emb = tensors[model.spec.embedding_name]
            if tuple(head.shape) != tuple(emb.shape) or not torch.equal(
                    head.to(device=emb.device, dtype=emb.dtype), emb):
                raise WeightError(folder, [], [], [
                    "lm_head.weight: the configuration ties the head to the embedding table, but the stored "
                    "head differs from it"])
        model.bind(tensors)
    finally:
        for f in files:
            f.close()
