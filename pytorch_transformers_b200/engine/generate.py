"""The generation loop above the step function.

Requests are served in batches: the prompts of a batch (of unequal lengths) run in one step,
then every live sequence advances by one token per step. A sequence that meets a stop token or
its budget of new tokens leaves the batch at once, its slot and pages go back to the cache and
the following steps are smaller; when a batch is done the next one starts, on the same cache.
The reference keeps finished rows in the batch and pads them until all rows are done
(src/transformers/generation/utils.py:3209, 3283, 3290-3291); the tokens that come out are
the same.

The loop knows nothing of devices: it drives a *stepper* (open / step / close) and a
*selector* (logits -> tokens), so its decisions are tested on the CPU with stand-ins.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, List, Optional, Protocol, Sequence

from ..config.generation import GenerationConfig


class Stepper(Protocol):
    def open(self) -> int: ...
    def close(self, slot: int) -> None: ...
    def step(self, slots: Sequence[int], token_lists: Sequence[Sequence[int]]): ...
    # optional: prepare(slots) builds the next step of one token each ahead of time;
    #           step_ahead(slots, device_tokens) runs that step with token ids that only the device knows yet
    #           (returns None if it cannot: the loop then waits for the tokens and calls step)


class Selector(Protocol):
    def select(self, logits, request_ids, step, histories=None, suppress_stop=False) -> List[int]: ...
    # optional: begin(...) launches the selection, finish(handle) waits for its tokens,
    #           device_tokens(handle) is where the device finds them before the host does


@dataclasses.dataclass
class RequestResult:
    prompt: List[int]
    tokens: List[int]                      # new tokens, a stop token included as the last one
    finish_reason: str = ""                # "stop" or "length"
    logits: Optional[list] = None          # per new token, the float32 logits row it was chosen from


def plan_batches(n_requests: int, max_batch: int) -> List[List[int]]:
    """Requests in order, ``max_batch`` at a time."""
    if max_batch < 1:
        raise ValueError("max_batch must be >= 1")
    return [list(range(i, min(i + max_batch, n_requests))) for i in range(0, n_requests, max_batch)]


def run_generation(stepper: Stepper, selector: Selector, prompts: Sequence[Sequence[int]],
                   options: GenerationConfig, budget: int, max_batch: int,
                   on_token: Optional[Callable[[int, int], None]] = None,
                   keep_logits: bool = False,
                   on_step: Optional[Callable[[dict], None]] = None) -> List[RequestResult]:
    """Generate up to ``budget`` tokens for every prompt; returns results in the prompts' order.

    ``on_token(request_index, token)`` is called for every new token as it is chosen, and
    ``on_step({request_index: token})`` once per step with all of the step's new tokens (the
    reference's streamer gets a step's tokens in one call, utils.py:3287-3288)."""
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {i} is empty: a sequence needs at least one token to start from")
    if budget < 1:
        raise ValueError("the budget of new tokens must be >= 1")
    stop = set(options.eos_ids())
    min_new = int(options.min_new_tokens or 0)
    results = [RequestResult(prompt=list(p), tokens=[]) for p in prompts]
    # a stepper that can prepare a step ahead and a selector that can run without the host waiting
    can_overlap = all(hasattr(selector, n) for n in ("begin", "finish")) and hasattr(stepper, "prepare")
    can_pipeline = can_overlap and hasattr(stepper, "step_ahead") and hasattr(selector, "device_tokens")
    for batch in plan_batches(len(prompts), max_batch):
        held = set()
        live = []
        try:
            for r in batch:
                slot = stepper.open()
                held.add(slot)
                live.append((r, slot))
            logits = stepper.step([s for _, s in live], [results[r].prompt for r, _ in live])
            for t in range(budget):
                req_ids = [r for r, _ in live]
                slots = [s for _, s in live]
                histories = ([results[r].prompt + results[r].tokens for r in req_ids]
                             if options.repetition_penalty != 1.0 else None)
                suppress = bool(stop) and t < min_new
                ahead = None
                if can_overlap:
                    # The selection runs on the device without the host waiting. Meanwhile the host builds
                    # the next step of one token each for the sequences that are live now and, if the
                    # stepper can take its tokens from the device, launches it at once: the device then
                    # goes from this step's selection straight into the next step, and the host reads the
                    # tokens (for the results, the stop tokens and the callback) while that step runs.
                    # A sequence that turns out to end here was in that step for nothing: its row is
                    # dropped.
                    pending = selector.begin(logits, req_ids, t, histories=histories, suppress_stop=suppress)
                    if t + 1 < budget:
                        stepper.prepare(slots)
                        if can_pipeline:
                            ahead = stepper.step_ahead(slots, selector.device_tokens(pending))
                    chosen = selector.finish(pending)
                else:
                    chosen = selector.select(logits, req_ids, t, histories=histories, suppress_stop=suppress)
                still, kept_rows = [], []
                for row, ((r, slot), tok) in enumerate(zip(live, chosen)):
                    res = results[r]
                    res.tokens.append(int(tok))
                    if keep_logits:
                        if res.logits is None:
                            res.logits = []
                        res.logits.append(logits[row])
                    if on_token is not None:
                        on_token(r, int(tok))
                    if int(tok) in stop and t >= min_new:
                        res.finish_reason = "stop"
                    elif len(res.tokens) >= budget:
                        res.finish_reason = "length"
                    if res.finish_reason:
                        held.discard(slot)
                        stepper.close(slot)       # the slot is free for the next batch right away
                    else:
                        still.append((r, slot))
                        kept_rows.append(row)
                if on_step is not None:
                    on_step({r: int(tok) for (r, _), tok in zip(live, chosen)})
                n_before = len(live)
                live = still
                if not live:
                    break
                if ahead is not None:
                    logits = ahead if len(live) == n_before else ahead[kept_rows]
                else:
                    logits = stepper.step([s for _, s in live], [[results[r].tokens[-1]] for r, _ in live])
        finally:
            for slot in sorted(held):             # only after an error: what is still open goes back
                stepper.close(slot)
    return results
