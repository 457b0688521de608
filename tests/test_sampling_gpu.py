"""The selection kernel against the plain filters: greedy, temperature, top-k, top-p, min-p,
repetition penalty, suppression of stop tokens, and draws that do not depend on the batch."""
import numpy as np
import pytest
import torch

import plain_falcon as plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from pytorch_transformers_b200 import kernels
    kernels.lib()
    return kernels


def select(K, logits, n_draws=1, **opt):
    """Tokens [n_draws, rows] chosen from `logits` (draw i uses counter i)."""
    rows, vocab = logits.shape
    work = torch.empty_like(logits)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    streams = opt.pop("streams", torch.arange(rows, dtype=torch.int64)).cuda()
    res = []
    for i in range(n_draws):
        counters = torch.full((rows,), i, dtype=torch.int64).cuda()
        K.sample(logits, work, out, streams=streams, counters=counters, **opt)
        res.append(out.clone())
    return torch.stack(res).cpu()


@pytest.mark.parametrize("vocab", [5, 333, 1000, 65024])
def test_greedy_is_argmax_lowest_index_on_ties(K, vocab):
    g = torch.Generator().manual_seed(vocab)
    logits = torch.randn(7, vocab, generator=g).cuda()
    logits[3, vocab // 2] = logits[3].max() + 1
    logits[4, 2] = logits[4, vocab - 1] = 50.0
    before = logits.clone()
    got = select(K, logits, do_sample=False)[0]
    assert got.tolist() == logits.argmax(-1).tolist() and got[4] == 2
    assert torch.equal(logits, before)               # the logits themselves are left alone


def empirical(tokens, vocab):
    return np.bincount(tokens.numpy().ravel(), minlength=vocab) / tokens.numel()


def test_temperature_sampling_follows_softmax(K):
    vocab, n = 12, 20000
    logits = torch.linspace(-2, 2, vocab)[None].cuda().contiguous()
    for temp in (0.5, 1.0, 2.0):
        toks = select(K, logits, n_draws=n, do_sample=True, temperature=temp, top_k=0)
        p = plain.temperature_probs(logits[0].cpu(), temp).numpy()
        err = np.abs(empirical(toks, vocab) - p)
        assert err.max() < 4 * np.sqrt(p.max() / n) + 1e-3, (temp, err.max())


def test_filters_keep_what_the_plain_filters_keep(K):
    g = torch.Generator().manual_seed(1)
    vocab, n = 40, 3000
    logits = (torch.randn(1, vocab, generator=g) * 2).cuda()
    lg = logits[0].cpu()
    cases = [
        (dict(top_k=5), plain.top_k_filter(lg, 5)),
        (dict(top_k=0, top_p=0.7), plain.top_p_filter(lg, 0.7)),
        (dict(top_k=0, top_p=0.2), plain.top_p_filter(lg, 0.2)),
        (dict(top_k=10, top_p=0.9, temperature=0.7), plain.top_p_filter(plain.top_k_filter(lg / 0.7, 10), 0.9)),
        (dict(top_k=0, min_p=0.1), lg.masked_fill(torch.softmax(lg, -1) < 0.1 * torch.softmax(lg, -1).max(), float("-inf"))),
        (dict(top_k=1), plain.top_k_filter(lg, 1)),
    ]
    for opt, kept in cases:
        toks = select(K, logits, n_draws=n, do_sample=True, **opt)
        allowed = set(torch.nonzero(torch.isfinite(kept)).ravel().tolist())
        seen = set(toks.ravel().tolist())
        assert seen <= allowed, (opt, seen - allowed)
        p = torch.softmax(kept.double(), -1).numpy()
        likely = {i for i in allowed if p[i] > 0.02}
        assert likely <= seen, (opt, likely - seen)
        assert np.abs(empirical(toks, vocab) - p).max() < 0.04


def test_repetition_penalty_and_suppression(K):
    logits = torch.tensor([[1.0, 3.0, 2.0, -1.0, 0.5, 2.9]]).cuda()
    hist = torch.tensor([[1, 1, 3, 0]], dtype=torch.int32).cuda()     # token 1 twice: penalised once
    hlen = torch.tensor([3], dtype=torch.int32).cuda()                # the 4th entry is not history
    ref = plain.repetition_penalty(logits[0].cpu(), [1, 1, 3], 2.0)
    got = select(K, logits, do_sample=False, repetition_penalty=2.0, history=hist, history_len=hlen)[0]
    assert got.item() == ref.argmax().item() == 5
    sup = torch.tensor([5, 1], dtype=torch.int32).cuda()
    assert select(K, logits, do_sample=False, suppress=sup)[0].item() == 2


def test_draws_depend_on_seed_request_and_step_not_on_the_batch(K):
    g = torch.Generator().manual_seed(2)
    logits = torch.randn(6, 500, generator=g).cuda()
    streams = torch.tensor([10, 11, 12, 13, 14, 15])
    full = select(K, logits, n_draws=8, do_sample=True, top_k=0, seed=5, streams=streams)
    sub = select(K, logits[[4, 1]].contiguous(), n_draws=8, do_sample=True, top_k=0, seed=5, streams=streams[[4, 1]])
    assert torch.equal(sub, full[:, [4, 1]])
    other = select(K, logits, n_draws=8, do_sample=True, top_k=0, seed=6, streams=streams)
    assert not torch.equal(other, full)
    assert len(set(full[:, 0].tolist())) > 1          # the step counter moves the draw


def test_bad_options_are_refused(K):
    from pytorch_transformers_b200.kernels import KernelError
    logits = torch.zeros(1, 10).cuda()
    for bad in (dict(temperature=0.0), dict(top_p=0.0), dict(top_p=1.5), dict(min_p=2.0)):
        with pytest.raises(KernelError):
            select(K, logits, do_sample=True, **bad)


def test_sampling_through_generate(tmp_path):
    import pytorch_transformers_b200 as ptb
    import tiny_models as tm
    model = ptb.AutoModelForCausalLM.from_pretrained(tm.tiny_folder(str(tmp_path), "A"), dtype="float32")
    prompts = tm.prompts("A", (4, 9, 6), seed=3)
    kw = dict(max_new_tokens=6, do_sample=True, temperature=1.5, top_k=0, eos_token_id=None)
    a = model.generate(prompts, seed=1, **kw)
    b = model.generate(prompts, seed=1, max_batch_size=1, **kw)       # one by one: same draws
    c = model.generate(prompts, seed=2, **kw)
    assert a == b and a != c
    two = model.generate(prompts[:1], seed=1, num_return_sequences=2, **kw)
    assert len(two) == 2 and two[0] != two[1] and two[0] == a[0]
    # top_k=1 sampling is greedy
    assert model.generate(prompts, max_new_tokens=5, do_sample=True, top_k=1, eos_token_id=None) == \
        model.generate(prompts, max_new_tokens=5, eos_token_id=None)


def draws_of_one_row(K, row, rows=4096, n_draws=64, **opt):
    """rows x n_draws draws from one row of logits (each copy of the row has a stream of its own)."""
    logits = row[None].expand(rows, -1).contiguous().cuda()
    return select(K, logits, n_draws=n_draws, do_sample=True, **opt)


def check_kept_set(toks, kept, exact_above=25.0):
    """No token outside the plain filter's set; every token of the set that is expected at least
    `exact_above` times is drawn; the rarest tenth of the set gets its share of the draws."""
    allowed = torch.isfinite(kept)
    counts = torch.bincount(toks.ravel(), minlength=kept.numel())
    assert counts[~allowed].sum() == 0, torch.nonzero(counts * ~allowed).ravel()[:10]
    p = torch.softmax(kept.double(), -1)
    expected = p * toks.numel()
    assert (counts[expected >= exact_above] > 0).all()
    order = torch.argsort(p + (~allowed) * 2.0)          # allowed tokens first, rarest first
    tail = order[: max(1, int(allowed.sum()) // 10)]
    want = float(expected[tail].sum())
    assert abs(float(counts[tail].sum()) - want) < 5 * want ** 0.5 + 3, (float(counts[tail].sum()), want)


@pytest.mark.parametrize("vocab,scale,opt", [
    (65024, 3.0, dict(top_k=50)),                      # the threads' maxima bound the candidates
    (70001, 3.0, dict(top_k=50, top_p=0.8)),           # a width that is no multiple of four
    (65024, 1.0, dict(top_k=2000)),                    # more candidates than the block holds
    (2000, 0.3, dict(top_k=0, top_p=0.9)),             # flat: the cut lies far below the first candidates
    (70001, 0.5, dict(top_k=0, top_p=0.9)),            # flat and wide: several narrowing passes
    (65024, 6.0, dict(top_k=0, top_p=0.9)),            # peaked: the cut lies among the first candidates
    (65024, 2.0, dict(top_k=3000, top_p=0.7)),         # top-p below a top-k that does not fit the block
    (5000, 2.0, dict(top_k=0, min_p=0.05)),
    (65024, 2.0, dict(top_k=0, temperature=0.7)),
])
def test_filters_on_wide_rows(K, vocab, scale, opt):
    g = torch.Generator().manual_seed(vocab + int(scale * 10))
    lg = torch.randn(vocab, generator=g) * scale
    kept = lg / opt.get("temperature", 1.0)
    if opt.get("top_k", 0) > 0:
        kept = plain.top_k_filter(kept, opt["top_k"])
    if opt.get("top_p", 1.0) < 1.0:
        kept = plain.top_p_filter(kept, opt["top_p"])
    if opt.get("min_p", 0.0) > 0.0:
        pr = torch.softmax(kept, -1)
        kept = kept.masked_fill(pr < opt["min_p"] * pr.max(), float("-inf"))
    check_kept_set(draws_of_one_row(K, lg, **opt), kept)


def test_top_k_keeps_all_ties_with_the_last_value_even_when_they_overflow_the_block(K):
    g = torch.Generator().manual_seed(9)
    lg = torch.rand(5000, generator=g)               # below 1
    perm = torch.randperm(5000, generator=g)
    lg[perm[:1500]] = 2.0
    lg[perm[1500:1505]] = 3.0
    toks = draws_of_one_row(K, lg, top_k=10)
    check_kept_set(toks, plain.top_k_filter(lg, 10))
    assert set(toks.ravel().tolist()) == set(perm[:1505].tolist())
