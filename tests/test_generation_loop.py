"""The generation loop's decisions, with stand-ins for the model and the selector (no GPU)."""
import pytest
import torch

from pytorch_transformers_b200.config import GenerationConfig
from pytorch_transformers_b200.engine import plan_batches, run_generation

VOCAB = 50


class FakeStepper:
    """A 'model' whose next token is (last token + 1) % VOCAB; records every call."""

    def __init__(self, max_slots=4):
        self.free = list(range(max_slots))
        self.length = {}
        self.calls = []
        self.closed = []

    def open(self):
        if not self.free:
            raise RuntimeError("no slot")
        s = min(self.free)
        self.free.remove(s)
        self.length[s] = 0
        return s

    def close(self, slot):
        assert slot in self.length, "slot closed twice"
        del self.length[slot]
        self.free.append(slot)
        self.closed.append(slot)

    def step(self, slots, token_lists):
        self.calls.append((list(slots), [list(t) for t in token_lists]))
        logits = torch.zeros(len(slots), VOCAB)
        for r, (s, toks) in enumerate(zip(slots, token_lists)):
            assert s in self.length
            self.length[s] += len(toks)
            logits[r, (toks[-1] + 1) % VOCAB] = 5.0
        return logits


class ArgmaxSelector:
    def __init__(self, stop=()):
        self.stop = list(stop)
        self.seen = []

    def select(self, logits, request_ids, step, histories=None, suppress_stop=False):
        self.seen.append((list(request_ids), step, suppress_stop))
        lg = logits.clone()
        if suppress_stop:
            lg[:, self.stop] = float("-inf")
        return lg.argmax(-1).tolist()


def test_plan_batches():
    assert plan_batches(7, 3) == [[0, 1, 2], [3, 4, 5], [6]]
    assert plan_batches(2, 5) == [[0, 1]]
    with pytest.raises(ValueError):
        plan_batches(3, 0)


def test_unequal_prompts_one_prefill_then_single_tokens():
    st, sel = FakeStepper(), ArgmaxSelector()
    prompts = [[1, 2, 3], [10], [20, 21]]
    res = run_generation(st, sel, prompts, GenerationConfig(), budget=4, max_batch=8)
    assert [r.tokens for r in res] == [[4, 5, 6, 7], [11, 12, 13, 14], [22, 23, 24, 25]]
    assert all(r.finish_reason == "length" for r in res)
    assert st.calls[0] == ([0, 1, 2], prompts)                 # all prompts in one step
    assert all(all(len(t) == 1 for t in c[1]) for c in st.calls[1:])
    assert len(st.calls) == 4                                  # no step after the last token
    assert st.length == {} and sorted(st.closed) == [0, 1, 2]


def test_stop_token_ends_a_sequence_and_the_batch_shrinks():
    st, sel = FakeStepper(), ArgmaxSelector()
    opts = GenerationConfig(eos_token_id=[12, 40])
    res = run_generation(st, sel, [[1, 2, 3], [10], [38]], opts, budget=5, max_batch=8)
    assert res[1].tokens == [11, 12] and res[1].finish_reason == "stop"      # the stop token is kept
    assert res[2].tokens == [39, 40] and res[2].finish_reason == "stop"
    assert res[0].tokens == [4, 5, 6, 7, 8] and res[0].finish_reason == "length"
    assert [c[0] for c in st.calls] == [[0, 1, 2], [0, 1, 2], [0], [0], [0]]  # later steps are smaller
    assert st.closed[:2] == [1, 2]


def test_batches_one_after_another_reuse_slots():
    st, sel = FakeStepper(max_slots=2), ArgmaxSelector()
    prompts = [[i] for i in range(5)]
    res = run_generation(st, sel, prompts, GenerationConfig(), budget=2, max_batch=2)
    assert [r.tokens for r in res] == [[i + 1, i + 2] for i in range(5)]
    prefill_slots = [c[0] for c in st.calls if len(c[1][0]) == 1 and c[1][0][0] < 5 and len(c[0]) in (1, 2)][::2]
    assert prefill_slots == [[0, 1], [0, 1], [0]]
    assert st.length == {}


def test_min_new_tokens_suppresses_the_stop_token():
    st, sel = FakeStepper(), ArgmaxSelector(stop=[11])
    opts = GenerationConfig(eos_token_id=11, min_new_tokens=3)
    res = run_generation(st, sel, [[10]], opts, budget=6, max_batch=1)
    assert [s[2] for s in sel.seen[:4]] == [True, True, True, False]
    assert 11 not in res[0].tokens[:3]


def test_streaming_callback_and_logits():
    st, sel = FakeStepper(), ArgmaxSelector()
    seen = []
    res = run_generation(st, sel, [[1], [7, 8]], GenerationConfig(), budget=2, max_batch=2,
                         on_token=lambda r, t: seen.append((r, t)), keep_logits=True)
    assert seen == [(0, 2), (1, 9), (0, 3), (1, 10)]
    assert len(res[0].logits) == 2 and res[0].logits[0].argmax().item() == 2


def test_errors_leave_no_slot_open():
    st, sel = FakeStepper(), ArgmaxSelector()
    with pytest.raises(ValueError, match="prompt 1 is empty"):
        run_generation(st, sel, [[1], []], GenerationConfig(), budget=2, max_batch=2)

    class Boom(FakeStepper):
        def step(self, slots, token_lists):
            if len(self.calls) == 2:
                raise RuntimeError("boom")
            return super().step(slots, token_lists)

    st = Boom()
    with pytest.raises(RuntimeError, match="boom"):
        run_generation(st, sel, [[1], [2]], GenerationConfig(), budget=5, max_batch=2)
    assert st.length == {} and sorted(st.free) == [0, 1, 2, 3]


class PreparingStepper(FakeStepper):
    """A stepper that can build a step ahead of time; it records what it was asked to prepare."""

    def __init__(self, max_slots=4):
        super().__init__(max_slots)
        self.prepared = []

    def prepare(self, slots):
        assert all(s in self.length for s in slots), "a step was prepared for a slot that is not open"
        self.prepared.append((len(self.calls), list(slots)))


class TwoPhaseSelector(ArgmaxSelector):
    """A selector whose selection can run while the host does something else."""

    def __init__(self, stop=()):
        super().__init__(stop)
        self.open_handle = None

    def begin(self, logits, request_ids, step, histories=None, suppress_stop=False):
        assert self.open_handle is None
        self.open_handle = self.select(logits, request_ids, step, histories, suppress_stop)
        return "handle"

    def finish(self, handle):
        assert handle == "handle"
        out, self.open_handle = self.open_handle, None
        return out


def test_the_next_step_is_prepared_while_the_selection_runs_and_changes_no_token():
    prompts = [[3, 4], [10], [20, 21, 22]]
    opts = GenerationConfig(eos_token_id=[13])                       # request 1 stops at its third token
    plain_results = run_generation(FakeStepper(), ArgmaxSelector([13]), prompts, opts, 5, 3)
    stepper, selector = PreparingStepper(), TwoPhaseSelector([13])
    results = run_generation(stepper, selector, prompts, opts, 5, 3)
    assert [r.tokens for r in results] == [r.tokens for r in plain_results]
    assert [r.finish_reason for r in results] == ["length", "stop", "length"]
    assert selector.open_handle is None
    # a step was prepared after every selection but the last one of the budget, for the sequences live
    # at that moment (request 1 among them at the step at which it ends: that preparation is wasted,
    # the step that follows names other slots)
    assert [n for n, _ in stepper.prepared] == [1, 2, 3, 4]
    assert stepper.prepared[0][1] == [0, 1, 2] and stepper.prepared[2][1] == [0, 1, 2]
    assert stepper.prepared[3][1] == [0, 2]
    assert stepper.calls[2][0] == [0, 1, 2] and stepper.calls[3][0] == [0, 2]
    # a stepper or a selector without the optional methods is driven the plain way
    results = run_generation(FakeStepper(), TwoPhaseSelector([13]), prompts, opts, 5, 3)
    assert [r.tokens for r in results] == [r.tokens for r in plain_results]


class PipelinedStepper(PreparingStepper):
    """A stepper that can also run the prepared step with token ids that only the 'device' knows: here
    the device is a list that the selector fills."""

    def __init__(self, max_slots=4, refuse_every=0):
        super().__init__(max_slots)
        self.ahead = []
        self.refuse_every = refuse_every

    def step_ahead(self, slots, device_tokens):
        assert self.prepared and self.prepared[-1] == (len(self.calls), list(slots)), "step_ahead without its preparation"
        if self.refuse_every and (len(self.ahead) + len(self.calls)) % self.refuse_every == 0:
            return None                                       # "no graph for this layout yet"
        self.ahead.append(list(slots))
        return self.step(slots, [[t] for t in device_tokens])


class DeviceSelectorFake(TwoPhaseSelector):
    def device_tokens(self, handle):
        return list(self.open_handle)          # on the device the tokens exist as soon as the kernel has run


@pytest.mark.parametrize("refuse_every", [0, 3])
def test_steps_launched_ahead_with_device_tokens_give_the_same_results(refuse_every):
    prompts = [[3, 4], [10], [20, 21, 22], [40], [47, 48]]
    opts = GenerationConfig(eos_token_id=[13, 49], min_new_tokens=2)     # requests 1 and 4 stop early
    want = run_generation(FakeStepper(), ArgmaxSelector([13, 49]), prompts, opts, 6, 3, keep_logits=True)
    seen = []
    stepper, selector = PipelinedStepper(refuse_every=refuse_every), DeviceSelectorFake([13, 49])
    got = run_generation(stepper, selector, prompts, opts, 6, 3, keep_logits=True,
                         on_token=lambda r, tok: seen.append((r, tok)))
    assert [r.tokens for r in got] == [r.tokens for r in want]
    assert [r.finish_reason for r in got] == [r.finish_reason for r in want]
    for a, b in zip(got, want):
        assert len(a.logits) == len(b.logits) and all(torch.equal(x, y) for x, y in zip(a.logits, b.logits))
    assert [tok for r, tok in seen if r == 1] == got[1].tokens
    assert stepper.ahead                                                  # steps did run ahead
    # request 1 ended at its third token ([11, 12, 13]); the step launched ahead of that selection still had
    # its slot in it, and its row was dropped: the steps after it name the other two slots only
    assert got[1].tokens == [11, 12, 13] and got[1].finish_reason == "stop"
    first_batch = [c[0] for c in stepper.calls[1:] if 1 in c[0] or c[0] == [0, 2]]
    assert first_batch.count([0, 1, 2]) == 3 and [0, 2] in first_batch
    assert sorted(stepper.free) == [0, 1, 2, 3] and not stepper.length    # every slot came back once
