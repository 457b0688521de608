"""Part interfaces, the part registry, and the data that describes a model as parts.

A model is data: a ``ModelSpec`` names an embedding, a list of blocks, the order in which the
blocks run (``schedule``), a final norm and an output head. Every block is a ``PartSpec`` that
names a registered block kind and holds the ``PartSpec`` of its mixer, feed-forward and norms.
A part gets its sizes and constants as constructor parameters and never learns which model it
is in: the architecture's builder (models/) turns a configuration into specs and supplies the
checkpoint's tensor names for the part's logical parameter names.

Families and what each must provide (all tensors are on the device; ``ctx`` is the
engine.batch.StepContext of the running step; ``x`` is [tokens, hidden] in the model dtype):

* ``norm``:          ``forward(x) -> y``; optionally ``forward_pair(x, other) -> (y, y_other)``.
* ``position``:      ``rotation() -> (inv_freq float32 [pairs], pairs) | None`` and
                     ``score_bias() -> slopes float32 [heads] | None``.
* ``mixer``:         ``forward(x, ctx, entry) -> y``; ``cache_need() -> CacheNeed | None``;
                     ``state_need() -> StateNeed | None``. ``entry`` is the ScheduleEntry being
                     run: it names the cache entry to read and whether to write it. Optional:
                     ``planner()`` (per-step arrays of its own) and ``runs_beside(ctx)``.
* ``feed_forward``:  ``forward(x, ctx) -> y``.
* ``block``:         ``forward(x, ctx, entry) -> x'`` from its child parts; ``x`` and ``x'`` may be a
                     ``DeferredSum`` (two terms whose sum the next norm forms); ``resolve`` gives the tensor.

Every part declares its parameters in ``param_decls()`` (logical name -> ParamDecl) and
receives them in ``bind(tensors)``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

FAMILIES = ("norm", "position", "mixer", "feed_forward", "block")
_REGISTRY: Dict[str, Dict[str, type]] = {f: {} for f in FAMILIES}


def register_part(family: str, kind: str, cls: Optional[type] = None):
    """Register a part class under (family, kind). Usable as a decorator."""
    if family not in _REGISTRY:
        raise ValueError(f"unknown part family {family!r} (families: {', '.join(FAMILIES)})")

    def _do(c: type) -> type:
        _REGISTRY[family][kind] = c
        return c

    return _do if cls is None else _do(cls)


def part_class(family: str, kind: str) -> type:
    try:
        return _REGISTRY[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(family, {}))) or "none"
        raise ValueError(f"no {family} part of kind {kind!r} is registered (registered: {known})") from None


@dataclasses.dataclass(frozen=True)
class ParamDecl:
    """A parameter of a part.

    ``role`` decides how it is held on the device: ``"matrix"`` tensors follow the model dtype
    (bfloat16 or float32); ``"vector"`` tensors (gains, biases) are held in float32, which is
    lossless for any stored dtype, so a vector stored in 32-bit stays 32-bit; ``"int"`` tensors
    are int32 tables. ``init`` names the law of the random-weights mode: ``normal`` is
    N(0, std), ``one_plus_normal`` is 1 + N(0, std).
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    std: float = 0.02


@dataclasses.dataclass
class PartSpec:
    """One part: registry kind, constructor parameters, child parts, checkpoint names.

    ``names`` maps the part's logical parameter names to tensor names of the checkpoint."""
    family: str
    kind: str
    params: Dict[str, Any] = dataclasses.field(default_factory=dict)
    children: Dict[str, "PartSpec"] = dataclasses.field(default_factory=dict)
    names: Dict[str, str] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(frozen=True)
class ScheduleEntry:
    """One run of a block. ``block`` indexes ModelSpec.blocks (a block may be named twice);
    ``cache_entry`` names the cache entry its mixer uses (entries are numbered over the whole
    schedule); with ``writes_cache=False`` the mixer only reads an entry that an earlier
    schedule entry wrote (one layer reading another layer's keys and values)."""
    block: int
    cache_entry: int
    writes_cache: bool = True


@dataclasses.dataclass
class ModelSpec:
    vocab_size: int
    hidden_size: int
    embedding_name: str
    blocks: List[PartSpec]
    final_norm: PartSpec
    head_name: Optional[str]          # None: the head shares the embedding table
    schedule: Optional[List[ScheduleEntry]] = None
    # what some architectures do between the table and the first block, and after the head (Falcon: nothing)
    embedding_scale: float = 1.0                  # x = table[ids] * embedding_scale
    embedding_norm: Optional[PartSpec] = None     # then a norm of the embeddings
    logit_scale: float = 1.0                      # logits = (rows @ head.T) * logit_scale

    def resolved_schedule(self) -> List[ScheduleEntry]:
        if self.schedule is not None:
            return list(self.schedule)
        return [ScheduleEntry(block=i, cache_entry=i) for i in range(len(self.blocks))]


@dataclasses.dataclass(frozen=True)
class CacheNeed:
    """What a mixer wants of the cache for one cache entry. ``kind`` is ``"full"`` (all keys
    and values of the sequence) or ``"window"`` (the last ``window`` of them)."""
    kind: str
    kv_heads: int
    head_dim: int
    window: int = 0


@dataclasses.dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-sequence state of a mixer for one cache entry: ``numel`` float32 values,
    zeroed when a sequence starts."""
    numel: int


@dataclasses.dataclass
class DeferredSum:
    """A residual stream whose last addition has not been done yet: the value is ``base + pending``.
    A block may hand this to the next block instead of a tensor when ``pending`` is still being
    computed on ``stream``; whoever needs the value waits for that stream and adds (the next
    block's norm does both in its own kernel). ``resolve`` gives the plain tensor."""
    base: Any
    pending: Any
    stream: Any = None

    def join(self, device) -> None:
        if self.stream is not None:
            torch.cuda.current_stream(device).wait_stream(self.stream)
            self.stream = None


def resolve(kernels, x):
    """The tensor that ``x`` stands for (``x`` itself, or the sum of a DeferredSum)."""
    if isinstance(x, DeferredSum):
        x.join(x.base.device)
        return kernels.residual(x.base, x.pending)
    return x


@dataclasses.dataclass
class BuildContext:
    """What parts need at construction: device, model dtype, and the kernel wrappers."""
    device: torch.device
    dtype: torch.dtype
    kernels: Any


class Part:
    """Base of every part. Subclasses set ``family`` through registration and implement
    ``param_decls`` and their family's methods.

    ``graph_safe``: the part's forward only launches work whose shapes and addresses depend on the
    step's layout (counts, widths, plans' facts), and reads everything else (slots, positions, pages)
    from the step's device arrays. Only then may a step be captured once and replayed as a CUDA
    graph; a part that loops over the step's host lists leaves it False and the model steps
    without graphs. The first step of a layout is run plainly and captured afterwards without
    running, every later one is a replay: a part's work is done once per step either way, so a
    part with per-sequence state needs no care for being run twice."""
    graph_safe = False

    def __init__(self, build: BuildContext, spec: PartSpec):
        self.build = build
        self.spec = spec
        self.children: Dict[str, Part] = {name: make_part(build, child) for name, child in spec.children.items()}

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for name, t in tensors.items():
            setattr(self, "p_" + name.replace(".", "_"), t)

    def planner(self):
        """An object with ``plan_key`` (a string) and ``plan(ctx) -> engine.batch.StepPlan`` if this part's
        kernels need per-step integer arrays or numbers beyond the step's own (tile lists, say); parts
        with the same ``plan_key`` share one plan per step, found as ``ctx.plan(plan_key)``. None: the part
        needs nothing."""
        return None

    def runs_beside(self, ctx) -> bool:
        """For mixers: may this step's mixer work run on a second stream (a second branch of a captured
        graph) beside the feed-forward's? A mixer says yes while its own kernels are small beside the
        feed-forward's read of its weights; the engine uses two branches only if every mixer agrees."""
        return False

    def walk(self):
        """This part and all parts below it."""
        yield self
        for c in self.children.values():
            yield from c.walk()


def make_part(build: BuildContext, spec: PartSpec) -> Part:
    cls = part_class(spec.family, spec.kind)
    return cls(build, spec, **spec.params)
