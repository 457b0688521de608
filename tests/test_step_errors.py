"""A step that cannot run as asked is refused on the host, before anything is launched or reserved:
the cache's lengths, pages and slots stay as they were. No GPU is needed: the checks sit in the
step's description (engine/batch.py) and in the cache's page accounting."""
import pytest
import torch

import tiny_models as tm

import pytorch_transformers_b200 as ptb
from pytorch_transformers_b200 import CacheFull, StepError
from pytorch_transformers_b200.cache.pool import CacheError


@pytest.fixture(scope="module")
def model():
    cfg = ptb.FalconConfig.from_dict(tm.config_dict("A"))
    return ptb.AutoModelForCausalLM.from_config(cfg, seed=1, dtype="float32", device="cpu")


def snapshot(cache):
    return ({s: (r.length, [list(p) for p in r.pages]) for s, r in cache.records.items()},
            [g.pool.in_use for g in cache.groups], cache.slots.in_use)


def held(cache):
    """A cache with two open sequences that already hold tokens (as two committed steps would leave it)."""
    a, b = cache.open(), cache.open()
    for slot, n in ((a, 70), (b, 5)):
        cache.reserve(slot, n)
        cache.commit(slot, n)
    return a, b


@pytest.mark.parametrize("slots, tokens, want, message", [
    ("aa", [[1], [2]], "last", "named twice"),
    ("ab", [[1], []], "last", "at least one token"),
    ("ab", [[1, 2, 3]], "last", "one item per sequence"),
    ("ab", [[1], [2]], [[0]], "one item per sequence"),
    ("", [], "last", "at least one sequence"),
    ("ab", [[1, 512], [2]], "last", "token id 512 is outside the vocabulary 0..511"),
    ("ab", [[1, -3], [2]], "last", "token id -3 is outside"),
    ("ab", [[1, 2], [2]], [[2], [0]], "wanted position 2 is outside the 2 tokens"),
    ("ab", [[1, 2], [2]], [[0], [-1]], "wanted position -1"),
    ("ab", [[1], [2]], "most", "want must be"),
])
def test_bad_arguments_raise_step_error_and_change_nothing(model, slots, tokens, want, message):
    cache = model.new_cache(64 * 8)
    a, b = held(cache)
    before = snapshot(cache)
    with pytest.raises(StepError, match=message):
        model.step(cache, [{"a": a, "b": b}[c] for c in slots], tokens, want)
    assert snapshot(cache) == before
    cache.check()


def test_a_slot_that_is_not_open_is_refused(model):
    cache = model.new_cache(64 * 8)
    a, b = held(cache)
    cache.close(b)
    before = snapshot(cache)
    with pytest.raises(CacheError, match="not open"):
        model.step(cache, [a, b], [[1], [2]])
    assert snapshot(cache) == before


def test_a_step_beyond_the_cache_is_refused_before_anything_is_reserved(model):
    cache = model.new_cache(64 * 4)          # four pages; the two sequences hold 2 + 1
    a, b = held(cache)
    before = snapshot(cache)
    # a needs no page for 58 more tokens, b needs one more for 60: fits exactly
    # together with 59 for a (one more page) it does not
    with pytest.raises(CacheFull, match="needs 2 more cache pages of 64 tokens but only 1 of 4 are free"):
        model.step(cache, [a, b], [[1] * 59, [2] * 60])
    assert snapshot(cache) == before
    cache.check()
    # a whole prompt that is too long for an empty cache
    fresh = model.new_cache(64 * 2)
    s = fresh.open()
    with pytest.raises(CacheFull):
        model.step(fresh, [s], [[3] * 129])
    assert fresh.length(s) == 0 and fresh.groups[0].pool.in_use == 0
    # more sequences than slots
    small = model.new_cache(64 * 8, max_slots=2)
    small.open(), small.open()
    with pytest.raises(CacheFull, match="sequence slot"):
        small.open()


def test_a_model_without_weights_says_so():
    cfg = ptb.FalconConfig.from_dict(tm.config_dict("A"))
    from pytorch_transformers_b200.config.registry import lookup_config
    from pytorch_transformers_b200.engine.model import CausalLM
    bare = CausalLM(lookup_config(cfg).spec_builder(cfg), cfg, device="cpu", dtype=torch.float32)
    cache = bare.new_cache(64)
    with pytest.raises(RuntimeError, match="no weights"):
        bare.step(cache, [cache.open()], [[1]])
