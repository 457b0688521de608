"""The description of one step: which tokens run, where they sit, where their cache pages are.

A step is a ragged batch: sequence ``b`` brings ``new[b]`` tokens that continue the
``past[b]`` tokens it already has in the cache. All index arrays are built on the host in one
int32 buffer and reach the device in one copy from page-locked memory; the kernels read them
through ``StepBatch`` (csrc/common.cuh). The reference pads prompts on the left and carries
``attention_mask``, ``position_ids`` and ``cache_position`` tensors instead
(src/transformers/generation/utils.py:349-481); here positions are arithmetic on lengths.

The step itself knows counts, positions and page tables only. What a kind of mixer needs
beyond that for its kernels (lists of tiles, say) comes from the mixer's *planner*: an object
with a ``plan_key`` and ``plan(ctx) -> StepPlan`` that the model collects from its parts. A
plan's integer arrays travel in the same buffer and copy as the step's own, and its ``facts``
(numbers that shape launches) are part of the layout.

The layout of the buffer depends only on the counts (tokens, sequences, wanted rows, width of
the page tables, and the plans' sizes and facts). A step of single tokens whose layout equals
an earlier one's can therefore reuse that step's device buffer: that is what lets a decode
step be replayed as a CUDA graph (``static`` below).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels as K
from ..cache.paged import PAGE, Cache


class PinnedRing:
    """A few page-locked host buffers used in turn for the step's index arrays, so that the copy
    to the device is asynchronous and no buffer is rewritten before its copy has run. ``fill`` puts
    a step's arrays into the next buffer (that can be done ahead of time, while the device is busy),
    ``send`` starts the copy to the device; ``stage`` does both."""

    def __init__(self, depth: int = 4):
        self.depth = depth
        self.buffers = [None] * depth
        self.views = [None] * depth     # the buffers as NumPy arrays
        self.events = [None] * depth
        self.next = 0

    def fill(self, packed: np.ndarray) -> int:
        i = self.next
        self.next = (i + 1) % self.depth
        buf = self.buffers[i]
        if buf is None or buf.numel() < packed.size:
            buf = torch.empty(max(4096, 2 * packed.size), dtype=torch.int32, pin_memory=True)
            self.buffers[i], self.views[i] = buf, buf.numpy()
            self.events[i] = torch.cuda.Event()
        else:
            self.events[i].synchronize()
        self.views[i][:packed.size] = packed
        return i

    def send(self, i: int, size: int, device: torch.device, into: Optional[torch.Tensor] = None) -> torch.Tensor:
        buf = self.buffers[i]
        if into is not None:
            into.copy_(buf[:size], non_blocking=True)
            dev = into
        else:
            dev = buf[:size].to(device, non_blocking=True)
        self.events[i].record(torch.cuda.current_stream(device))
        return dev

    def stage(self, packed: np.ndarray, device: torch.device, into: Optional[torch.Tensor] = None) -> torch.Tensor:
        if device.type != "cuda":
            t = torch.from_numpy(packed).to(device)
            if into is not None:
                into.copy_(t)
                return into
            return t
        return self.send(self.fill(packed), packed.size, device, into)


_RING = PinnedRing()


class StepError(ValueError):
    """A step that cannot be run as asked (bad slot, empty token list, token id out of range...)."""


@dataclasses.dataclass
class StepPlan:
    """What one planner adds to a step: ``arrays`` (name -> integer array, copied to the device with the
    step's own arrays and found in ``dev`` afterwards) and ``facts`` (name -> int, numbers that shape the
    kernels' launches and therefore belong to the step's layout)."""
    arrays: Dict[str, Any] = dataclasses.field(default_factory=dict)
    facts: Dict[str, int] = dataclasses.field(default_factory=dict)
    dev: Dict[str, torch.Tensor] = dataclasses.field(default_factory=dict)


class StepContext:
    """Everything a part may read about the running step.

    ``slots``, ``new``, ``past``: per sequence, on the host. ``dev[name]``: int32 device arrays
    (tokens, tok_seq, tok_pos, seq_start, seq_new, seq_past, slots, logits_at and one page table
    per storage group). ``batch_c[group]``: the StepBatch struct for the kernels.
    ``plans[plan_key]``: the StepPlan of each planner the step was built with.
    """

    def __init__(self, cache: Cache, slots: Sequence[int], token_lists: Sequence[Sequence[int]], vocab_size: int,
                 want: Sequence[Sequence[int]], planners: Sequence[Any] = (), page_bucket: int = 0,
                 defer: bool = False):
        if len(slots) != len(token_lists) or len(slots) != len(want):
            raise StepError("slots, token lists and wanted positions must have one item per sequence")
        if len(slots) == 0:
            raise StepError("a step needs at least one sequence")
        if len(set(slots)) != len(slots):
            raise StepError(f"a slot is named twice in one step: {list(slots)}")
        self.cache = cache
        self.side_stream = None     # set by the engine for steps of a few tokens (see parts/block.py)
        self._rope: dict = {}
        self.keep_alive: list = []  # tensors that must outlive the step's last kernel on another stream
        self.slots = [int(s) for s in slots]
        self.n_seqs = len(slots)
        self.new = [len(t) for t in token_lists]
        if min(self.new) < 1:
            raise StepError("every sequence of a step must bring at least one token")
        self.past = [cache.length(s) for s in self.slots]
        self.n_tokens = int(sum(self.new))
        self.is_decode = all(n == 1 for n in self.new)
        self.max_context = max(p + n for p, n in zip(self.past, self.new))

        tokens = np.fromiter((t for lst in token_lists for t in lst), dtype=np.int64, count=self.n_tokens)
        if tokens.min() < 0 or tokens.max() >= vocab_size:
            bad = int(tokens[(tokens < 0) | (tokens >= vocab_size)][0])
            raise StepError(f"token id {bad} is outside the vocabulary 0..{vocab_size - 1}")
        seq_start = np.zeros(self.n_seqs + 1, dtype=np.int64)
        np.cumsum(self.new, out=seq_start[1:])
        tok_seq = np.repeat(np.arange(self.n_seqs), self.new)
        tok_pos = np.concatenate([np.arange(p, p + n) for p, n in zip(self.past, self.new)])

        logits_at: List[int] = []
        for b, w in enumerate(want):
            for i in w:
                if not (0 <= int(i) < self.new[b]):
                    raise StepError(f"wanted position {i} is outside the {self.new[b]} tokens that sequence {b} brings")
                logits_at.append(int(seq_start[b]) + int(i))
        self.n_wanted = len(logits_at)

        # what the mixers' planners add (parts that share a plan_key share one plan); they see the
        # counts and positions above, and run before anything is reserved
        self.plans: Dict[str, StepPlan] = {}
        for planner in planners:
            if planner.plan_key not in self.plans:
                self.plans[planner.plan_key] = planner.plan(self)

        # page tables, one per storage group, padded to the longest (or to a whole bucket)
        cache.reserve_all(list(zip(self.slots, self.new)))
        tables = []
        for gi in range(len(cache.groups)):
            rows = [cache.pages(s, gi) for s in self.slots]
            width = max(1, max(len(r) for r in rows))
            if page_bucket:
                width = (width + page_bucket - 1) // page_bucket * page_bucket
            tab = np.full((self.n_seqs, width), -1, dtype=np.int64)
            for b, r in enumerate(rows):
                tab[b, :len(r)] = r
            tables.append(tab)
        self.table_widths: Tuple[int, ...] = tuple(t.shape[1] for t in tables)
        # pages that a sequence of this step may span: sizes the division of keys among blocks
        self.pages_hint = max(self.table_widths) if (page_bucket and tables) else (self.max_context + PAGE - 1) // PAGE

        parts = {"tokens": tokens, "tok_seq": tok_seq, "tok_pos": tok_pos, "seq_start": seq_start[:-1],
                 "seq_new": np.asarray(self.new), "seq_past": np.asarray(self.past),
                 "slots": np.asarray(self.slots), "logits_at": np.asarray(logits_at, dtype=np.int64)}
        for gi, tab in enumerate(tables):
            parts[f"pages{gi}"] = tab.reshape(-1)
        for key, plan in self.plans.items():
            for name, arr in plan.arrays.items():
                parts[f"plan.{key}.{name}"] = np.asarray(arr)
        offsets, total = {}, 0
        for name, arr in parts.items():
            offsets[name] = (total, arr.size)
            total += (arr.size + 3) // 4 * 4  # keep every array 16-byte aligned
        packed = np.zeros(max(total, 4), dtype=np.int32)
        for name, arr in parts.items():
            o, n = offsets[name]
            packed[o:o + n] = arr
        self.host = {name: packed[o:o + n] for name, (o, n) in offsets.items()}
        self.layout_key = (self.n_tokens, self.n_seqs, self.n_wanted, self.table_widths,
                           tuple((key, tuple(sorted(plan.facts.items())),
                                  tuple((n, np.asarray(a).size) for n, a in plan.arrays.items()))
                                 for key, plan in sorted(self.plans.items())))
        self.h2d_bytes = packed.nbytes
        self.packed_size = packed.size
        self._packed, self._offsets, self._tables = packed, offsets, tables
        self._pinned: Optional[int] = None      # index of the page-locked buffer that holds the arrays, if filled ahead
        self.dev: Dict[str, torch.Tensor] = {}
        self.batch_c: List[K.StepBatchC] = []
        if not defer:
            self.bind()

    def set_tokens(self, token_lists: Sequence[Sequence[int]], vocab_size: int) -> None:
        """Put other token ids into a step that was built ahead of time with placeholders (same counts);
        before ``bind``."""
        if [len(t) for t in token_lists] != self.new:
            raise StepError("the tokens do not fit the step that was prepared")
        tokens = np.fromiter((t for lst in token_lists for t in lst), dtype=np.int64, count=self.n_tokens)
        if tokens.min() < 0 or tokens.max() >= vocab_size:
            bad = int(tokens[(tokens < 0) | (tokens >= vocab_size)][0])
            raise StepError(f"token id {bad} is outside the vocabulary 0..{vocab_size - 1}")
        self.host["tokens"][:] = tokens
        if self._pinned is not None:        # the arrays are in page-locked memory already: the tokens follow
            o, n = self._offsets["tokens"]
            _RING.views[self._pinned][o:o + n] = tokens

    def fill_ahead(self) -> None:
        """Put the arrays into page-locked memory now (a step that is prepared ahead of time: only the
        tokens and the copy to the device are left for later)."""
        if self.cache.device.type == "cuda" and self._pinned is None:
            self._pinned = _RING.fill(self._packed)

    def _to_device(self, static: Optional[torch.Tensor]) -> torch.Tensor:
        if static is not None and static.numel() != self._packed.size:
            raise StepError("the static step buffer does not fit this step's layout")
        if self._pinned is not None:
            i, self._pinned = self._pinned, None
            return _RING.send(i, self._packed.size, self.cache.device, into=static)
        return _RING.stage(self._packed, self.cache.device, into=static)

    def refill(self, static: torch.Tensor) -> None:
        """Copy the index arrays into ``static``, the buffer that a captured graph of this layout reads:
        all that a replay needs (its kernels hold the addresses already)."""
        self._to_device(static)

    def bind(self, static: Optional[torch.Tensor] = None) -> None:
        """Copy the index arrays to the device, into a new buffer or into ``static`` (a buffer of
        exactly this layout's size that a captured graph reads), and make the views that the parts and
        the kernels read (``dev``, the plans' ``dev``, ``batch_c``)."""
        offsets, tables = self._offsets, self._tables
        dev = self._to_device(static)
        self.dev = {name: dev[o:o + n] for name, (o, n) in offsets.items()}
        for key, plan in self.plans.items():
            plan.dev = {name: self.dev[f"plan.{key}.{name}"] for name in plan.arrays}
        self.packed_dev = dev
        self.batch_c = []
        for gi, tab in enumerate(tables):
            c = K.StepBatchC()
            c.tok_seq, c.tok_pos = self.dev["tok_seq"].data_ptr(), self.dev["tok_pos"].data_ptr()
            c.seq_start, c.seq_new = self.dev["seq_start"].data_ptr(), self.dev["seq_new"].data_ptr()
            c.seq_past, c.pages = self.dev["seq_past"].data_ptr(), self.dev[f"pages{gi}"].data_ptr()
            c.pages_stride, c.n_tokens, c.n_seqs = tab.shape[1], self.n_tokens, self.n_seqs
            self.batch_c.append(c)

    def begin_forward(self) -> None:
        """Forget what an earlier forward pass over this step computed (a step that is captured as a
        graph runs once plainly and once under capture: the capture must contain every kernel)."""
        self._rope = {}
        self.keep_alive = []

    def rope(self, position_part):
        """(cos, sin) tables of this step's tokens for a rotary position part, computed once per step
        and set of constants (a part's ``rotation_key``; without one, per part) on first use (the reference computes them once per forward pass too,
        src/transformers/models/falcon/modeling_falcon.py:946); None for parts that do not rotate."""
        inv_freq = position_part.rotation() if position_part is not None else None
        if inv_freq is None:
            return None
        key = getattr(position_part, "rotation_key", None) or id(position_part)
        if key not in self._rope:
            self._rope[key] = K.rope_table(self.dev["tok_pos"], inv_freq)
        return self._rope[key]

    def plan(self, plan_key: str) -> StepPlan:
        try:
            return self.plans[plan_key]
        except KeyError:
            raise StepError(f"this step was built without the plan {plan_key!r}: pass the mixer's planner() to "
                            f"StepContext (plans of this step: {', '.join(sorted(self.plans)) or 'none'})") from None

    def tiles(self, rows: int):
        """(sequence, first token) of every tile of ``rows`` consecutive new tokens of one sequence."""
        seqs, firsts = [], []
        for b, n in enumerate(self.new):
            for q0 in range(0, n, rows):
                seqs.append(b)
                firsts.append(q0)
        return seqs, firsts

    def commit(self) -> None:
        for s, n in zip(self.slots, self.new):
            self.cache.commit(s, n)
