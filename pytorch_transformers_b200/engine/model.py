"""The model as the engine sees it: parts put together from a ModelSpec, and the step function.

``CausalLM.step`` is the one forward pass of the library: a ragged batch of sequences (whole
prompts, chunks of prompts or single tokens, in any mix) runs from the cache and returns
float32 logits at the wanted positions. Generation, trace replay and the benchmark all go
through it. It stands where ``FalconForCausalLM.forward`` stands in the reference
(src/transformers/models/falcon/modeling_falcon.py:1185-1254: embedding, blocks, ln_f, lm_head
on the last ``num_logits_to_keep`` positions), without padding or mask tensors.
"""
from __future__ import annotations

import gc
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from .. import kernels as K
from ..cache.paged import Cache
from ..parts.base import BuildContext, ModelSpec, ParamDecl, Part, make_part, resolve
from ..parts.linear import linear
from .batch import StepContext, StepError


class _StepSpan:
    """Context manager around a step's launches: two CUDA events and a record, if records are kept."""

    def __init__(self, model, kind: str, ctx: StepContext):
        self.model, self.kind, self.ctx = model, kind, ctx
        self.on = model.step_records is not None and model.device.type == "cuda"

    def __enter__(self):
        if self.on:
            self.begin = torch.cuda.Event(enable_timing=True)
            self.begin.record()

    def __exit__(self, *exc):
        if self.on and exc[0] is None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            ctx = self.ctx
            self.model.step_records.append({"kind": self.kind, "sequences": ctx.n_seqs, "tokens": ctx.n_tokens,
                                            "h2d_bytes": ctx.h2d_bytes, "begin": self.begin, "end": end})


class NoCollection:
    """No cyclic garbage collection inside: while a stream is being captured into a CUDA graph, an
    object that the collector happens to free then (a dropped cache with its graphs and page-locked
    buffers, a stream, an event) runs CUDA calls that are not allowed during a capture and void it.
    torch.cuda.graph collects what is garbage already when the capture begins; the collector goes back to
    what it was after."""

    def __enter__(self):
        self.was = gc.isenabled()
        gc.disable()

    def __exit__(self, *exc):
        if self.was:
            gc.enable()


class CausalLM:
    """A decoder-only language model built from parts."""

    def __init__(self, spec: ModelSpec, config, device="cuda", dtype=torch.bfloat16, kernels=K):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"model dtype must be float32 or bfloat16, got {dtype}")
        self.spec, self.config = spec, config
        self.device, self.dtype = torch.device(device), dtype
        self.build = BuildContext(device=self.device, dtype=dtype, kernels=kernels)
        self.blocks: List[Part] = [make_part(self.build, b) for b in spec.blocks]
        self.final_norm: Part = make_part(self.build, spec.final_norm)
        self.embedding_norm: Optional[Part] = (make_part(self.build, spec.embedding_norm)
                                               if spec.embedding_norm is not None else None)
        self.schedule = spec.resolved_schedule()
        for e in self.schedule:
            if not (0 <= e.block < len(self.blocks)):
                raise ValueError(f"schedule names block {e.block} but the model has {len(self.blocks)} blocks")
        writers = {e.cache_entry for e in self.schedule if e.writes_cache}
        for e in self.schedule:
            if not e.writes_cache and e.cache_entry not in writers:
                raise ValueError(f"schedule entry reads cache entry {e.cache_entry}, which no entry writes")
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.status = None  # device int32 word raised by kernels that clamp a bad index
        # replay steps of single tokens as CUDA graphs, if every part allows it
        self.use_graphs = all(p.graph_safe for top in self._top_parts() for p in top.walk())
        self.last_h2d_bytes = 0
        self.step_records: Optional[list] = None   # set by record_steps(True): one record per step
        self._side_stream = None
        # what the parts ask of every step: their planners (one per plan_key) and the mixers' word on streams
        self.planners, seen = [], set()
        for top in self._top_parts():
            for part in top.walk():
                planner = part.planner()
                if planner is not None and planner.plan_key not in seen:
                    seen.add(planner.plan_key)
                    self.planners.append(planner)
        self._mixers = [b.children["mixer"] for b in self.blocks if "mixer" in b.children]

    def _top_parts(self) -> List[Part]:
        return self.blocks + [self.final_norm] + ([self.embedding_norm] if self.embedding_norm is not None else [])

    # ------------------------------------------------------------------ parameters
    def param_table(self) -> Dict[str, Tuple[Optional[Part], str, ParamDecl]]:
        """Checkpoint tensor name -> (owning part, logical name, declaration)."""
        table: Dict[str, Tuple[Optional[Part], str, ParamDecl]] = {}
        v, h = self.spec.vocab_size, self.spec.hidden_size
        table[self.spec.embedding_name] = (None, "embedding", ParamDecl((v, h)))
        if self.spec.head_name is not None:
            table[self.spec.head_name] = (None, "head", ParamDecl((v, h)))
        for top in self._top_parts():
            for part in top.walk():
                for logical, decl in part.param_decls().items():
                    try:
                        name = part.spec.names[logical]
                    except KeyError:
                        raise ValueError(f"{part.spec.family} part {part.spec.kind!r} declares parameter "
                                         f"{logical!r} but its spec gives no checkpoint name for it") from None
                    if name in table:
                        raise ValueError(f"checkpoint tensor {name!r} is claimed by two parameters")
                    table[name] = (part, logical, decl)
        return table

    def device_dtype(self, decl: ParamDecl) -> torch.dtype:
        if decl.role == "vector":
            return torch.float32
        if decl.role == "int":
            return torch.int32
        return self.dtype

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Give every part its device tensors (keys are checkpoint names)."""
        per_part: Dict[int, Tuple[Part, Dict[str, torch.Tensor]]] = {}
        for name, (part, logical, decl) in self.param_table().items():
            t = tensors[name]
            if part is None:
                if logical == "embedding":
                    self.embedding = t
                else:
                    self.head = t
            else:
                per_part.setdefault(id(part), (part, {}))[1][logical] = t
        for part, group in per_part.values():
            part.bind(group)
        if self.spec.head_name is None:
            self.head = self.embedding  # one device buffer for the gather and the output product
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        tensors = [self.embedding, self.head]
        for top in self._top_parts():
            for part in top.walk():
                tensors += [getattr(part, a) for a in vars(part) if a.startswith("p_")]
        for t in tensors:
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def record_steps(self, on: bool = True) -> None:
        """Keep a record of every step from now on in ``step_records`` (a list of dicts: kind "prompt",
        "decode", "graph" or "ahead", sequences, tokens, bytes of index arrays copied, and two CUDA events
        around the step's launches) or stop keeping it. ``step_timings()`` turns the events into
        milliseconds. Off by default: an event pair per step is cheap but not free."""
        self.step_records = [] if on else None

    def step_timings(self) -> List[dict]:
        """The records of ``record_steps`` with ``device_ms`` (waits for the device)."""
        out = []
        for r in self.step_records or ():
            r["end"].synchronize()
            out.append({k: v for k, v in r.items() if k not in ("begin", "end")} |
                       {"device_ms": r["begin"].elapsed_time(r["end"])})
        return out

    def _recorded(self, kind: str, ctx: StepContext):
        """Context manager around a step's launches that adds a record when records are kept."""
        return _StepSpan(self, kind, ctx)

    def check_errors(self) -> None:
        """Raise if a kernel has reported trouble since the last check (synchronises): a row index that
        had to be clamped (a token id or a wanted row that was wrong on the device although the host
        had checked it, say in a buffer that a graph replays), or a bounded wait that ran out."""
        if self.status is not None:
            code = int(self.status.item())
            if code != 0:
                self.status.zero_()
                raise K.KernelError(f"a row index was out of range on the device (status {code}): the step's "
                                    "results are void")
        self.build.kernels.check_device_errors(self.device)

    # ------------------------------------------------------------------ cache
    def cache_needs(self):
        needs = []
        for e in self.schedule:
            if not e.writes_cache:
                continue
            mixer = self.blocks[e.block].children.get("mixer")
            needs.append((e.cache_entry, mixer.cache_need() if mixer else None,
                          mixer.state_need() if mixer else None))
        return needs

    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None) -> Cache:
        return Cache(self.cache_needs(), max_tokens, self.dtype, self.device, max_slots=max_slots)

    # ------------------------------------------------------------------ the step
    def step(self, cache: Cache, slots: Sequence[int], token_lists: Sequence[Sequence[int]],
             want: Union[str, Sequence[Sequence[int]]] = "last") -> torch.Tensor:
        """Run the given tokens of the given sequences as one batch from the cache.

        ``token_lists[b]`` are the next tokens of the sequence in ``slots[b]`` (its whole prompt,
        a chunk of it, or one token). ``want[b]`` lists the places among these tokens whose
        logits are returned ("last": the last token of each; "all": every token; "none").
        Returns float32 logits [wanted, vocab] in the order of the sequences and of ``want``.
        The sequences' lengths in the cache advance by the tokens run.
        """
        if self.embedding is None:
            raise RuntimeError("the model has no weights yet (load a checkpoint or initialise at random)")
        if isinstance(want, str):
            if want == "last":
                want = [[len(t) - 1] for t in token_lists]
            elif want == "all":
                want = [list(range(len(t))) for t in token_lists]
            elif want == "none":
                want = [[] for _ in token_lists]
            else:
                raise StepError(f"want must be 'last', 'all', 'none' or lists of positions, got {want!r}")
        single = all(len(t) == 1 for t in token_lists) and all(list(w) == [0] for w in want)
        ctx = self._take_prepared(cache, slots)     # whatever was prepared is used now or never
        if single and self.use_graphs and self.device.type == "cuda":
            if ctx is not None:
                ctx.set_tokens(token_lists, self.spec.vocab_size)
            else:
                ctx = StepContext(cache, slots, token_lists, self.spec.vocab_size, want, self.planners,
                                  page_bucket=self.GRAPH_PAGE_BUCKET, defer=True)
            return self._step_graph(cache, ctx)
        ctx = StepContext(cache, slots, token_lists, self.spec.vocab_size, want, self.planners)
        self.last_h2d_bytes = ctx.h2d_bytes     # index arrays copied to the device for this step
        with self._recorded("decode" if ctx.is_decode else "prompt", ctx):
            logits = self.forward(ctx)
        ctx.commit()
        return logits

    # A step of single tokens launches the same kernels with the same shapes as the one before it
    # when the batch size and the (bucketed) width of the page tables are unchanged: only the index
    # arrays differ. Such steps are captured once as a CUDA graph and replayed, which removes the
    # per-kernel launch cost of a few hundred launches per step. The graph reads its index arrays
    # from a buffer of its own that every replay refills.
    GRAPH_PAGE_BUCKET = 16
    MAX_GRAPHS = 16

    def prepare_next(self, cache: Cache, slots: Sequence[int]) -> bool:
        """Build ahead of time the step that will give each of ``slots`` one more token, while the device
        is still busy with the step before: positions, page tables (pages are reserved now) and plans
        need no token ids. The next ``step`` on this cache uses it if it is that step (same slots, same
        lengths, no sequence opened or closed since) and only puts the tokens in; any other step drops
        it. Returns whether a step was prepared (not without graphs, not when the cache is full)."""
        from ..cache.pool import CacheFull
        cache.__dict__.pop("_prepared_step", None)
        if not (self.use_graphs and self.device.type == "cuda") or len(slots) == 0:
            return False
        one = [[0]] * len(slots)
        try:
            ahead = StepContext(cache, slots, one, self.spec.vocab_size, one, self.planners,
                                page_bucket=self.GRAPH_PAGE_BUCKET, defer=True)
        except CacheFull:
            return False
        ahead.fill_ahead()
        cache.__dict__["_prepared_step"] = (id(self), cache.epoch, ahead)
        return True

    def _take_prepared(self, cache: Cache, slots: Sequence[int]) -> Optional[StepContext]:
        """The step that prepare_next built, if it is the step for ``slots`` now; whatever was prepared
        is used now or never."""
        prepared = cache.__dict__.pop("_prepared_step", None)
        if prepared is None:
            return None
        owner, epoch, ahead = prepared
        if (owner == id(self) and epoch == cache.epoch and ahead.slots == [int(s) for s in slots]
                and ahead.past == [cache.length(s) for s in ahead.slots]):
            return ahead
        return None

    def step_ahead(self, cache: Cache, slots: Sequence[int], device_tokens: torch.Tensor) -> Optional[torch.Tensor]:
        """Run the prepared step of one token each for ``slots`` with token ids that are on the device
        only (``device_tokens``: int32 [len(slots)], typically what the selection kernel of the step
        before wrote; they are read in stream order, so the selection need not have finished). Returns
        the logits as ``step`` does, or None when there is no prepared step for these slots or no
        captured graph for its layout yet: the caller then waits for the tokens and calls ``step``.
        The ids are not checked against the vocabulary here: they come from the selection kernel."""
        ctx = self._take_prepared(cache, slots)
        if ctx is None:
            return None
        entry = cache.__dict__.get("_step_graphs", {}).get((id(self), ctx.layout_key))
        if entry is None or device_tokens.dtype != torch.int32 or device_tokens.numel() < ctx.n_tokens:
            cache.__dict__["_prepared_step"] = (id(self), cache.epoch, ctx)     # still good for step()
            return None
        with self._recorded("ahead", ctx):
            ctx.refill(entry["static"])
            o, n = ctx._offsets["tokens"]
            entry["static"][o:o + n].copy_(device_tokens[:n], non_blocking=True)
            self.last_h2d_bytes = ctx.h2d_bytes
            entry["graph"].replay()
            out = entry["out"].clone()
        K.launches += entry["launches"]
        ctx.commit()
        return out

    def _step_graph(self, cache: Cache, ctx: StepContext) -> torch.Tensor:
        # graphs live on the cache they were captured for (they hold pointers into its storage)
        graphs = cache.__dict__.setdefault("_step_graphs", {})
        key = (id(self), ctx.layout_key)
        entry = graphs.get(key)
        if entry is None:
            static = torch.empty(ctx.packed_size, dtype=torch.int32, device=self.device)
            ctx.bind(static)
            # The first step of a layout runs plainly, and its result is what is returned: lazy
            # initialisations (and one-time set-up inside the library) happen here, outside the capture.
            # The capture that follows records the same launches without running them, so the step's
            # work, a mixer's update of its per-sequence state included, is done exactly once.
            with self._recorded("decode", ctx):
                first = self.forward(ctx)
            graph = torch.cuda.CUDAGraph()
            before = K.launches
            with NoCollection(), torch.cuda.graph(graph):
                out = self.forward(ctx)
            # kernels of this library that one replay launches (for the launch count of benchmarks);
            # the capture itself launched nothing
            entry = {"static": static, "graph": graph, "out": out, "launches": K.launches - before}
            K.launches = before
            while len(graphs) >= self.MAX_GRAPHS:
                graphs.pop(next(iter(graphs)))
            graphs[key] = entry
            self.last_h2d_bytes = ctx.h2d_bytes
            ctx.commit()
            return first
        with self._recorded("graph", ctx):
            ctx.refill(entry["static"])
            self.last_h2d_bytes = ctx.h2d_bytes
            entry["graph"].replay()
            out = entry["out"].clone()   # the graph's own output buffer is rewritten by the next replay
        K.launches += entry["launches"]
        ctx.commit()
        return out

    def _two_streams(self, ctx: StepContext) -> bool:
        """Mixer and feed-forward of a parallel block as two branches: only for steps of few rows (whose
        linear layers are weight streams), and only if every mixer of the model says that its work in
        this step is small beside such a stream (Part.runs_beside)."""
        k = self.build.kernels
        if self.device.type != "cuda" or ctx.n_tokens > k.WEIGHT_STREAM_MAX_ROWS or not self._mixers:
            return False
        return all(m.runs_beside(ctx) for m in self._mixers)

    def forward(self, ctx: StepContext) -> torch.Tensor:
        k = self.build.kernels
        ctx.begin_forward()
        if self._two_streams(ctx):
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(device=self.device)
            ctx.side_stream = self._side_stream
        x = k.gather_rows(ctx.dev["tokens"], self.embedding, self.status)
        if self.spec.embedding_scale != 1.0:
            k.scale_(x, self.spec.embedding_scale)
        if self.embedding_norm is not None:
            x = self.embedding_norm.forward(x)
        for entry in self.schedule:
            x = self.blocks[entry.block].forward(x, ctx, entry)   # a tensor, or a DeferredSum of two branches
        x = resolve(k, x)
        if ctx.n_wanted == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        rows = k.gather_rows(ctx.dev["logits_at"], x, self.status)
        rows = self.final_norm.forward(rows)
        return self.logits(rows)

    def logits(self, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits of normed rows: rows @ head.T (no bias, modeling_falcon.py:1168), times the
        spec's logit_scale where an architecture has one."""
        k = self.build.kernels
        if self.dtype == torch.float32:
            out = k.linear_f32(rows, self.head)
        elif k.skinny_linear_preferred(rows.shape[0], rows.shape[1], self.head.shape[0]):
            out = k.skinny_linear(rows, self.head, out_dtype=torch.float32)
        else:
            out = k.matmul_nt(rows, self.head, out_dtype=torch.float32)
        if self.spec.logit_scale != 1.0:
            k.scale_(out, self.spec.logit_scale)
        return out
