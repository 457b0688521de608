"""The engine against the plain implementation, in float32 and in bfloat16: each request alone
and whole; with the last 32 tokens one by one; in batches of unequal lengths whose shorter
requests end earlier, one batch after another on a small cache so that slots and pages are used
again; long decoding; the first tokens of a sequence; greedy generation through the entry point."""
import numpy as np
import pytest
import torch

import plain_falcon as plain
import tiny_models as tm

pytestmark = pytest.mark.gpu

CASES = {
    "A": ("A", {}), "B": ("B", {}), "C": ("C", {}), "D": ("D", {}), "E": ("E", {}), "F": ("F", {}), "G": ("G", {}),
    "A_sequential": ("A", {"parallel_attn": False}),
    "B_one_norm": ("B", {"num_ln_in_parallel_attn": 1}),
}
DTYPES = ["float32", "bfloat16"]
# float32: rounding of float32 sums against a float64 oracle, logits of magnitude ~1.
# bfloat16: weights and activations carry 8 bits; the oracle runs in float64 on the same
# bfloat16-rounded weights, so the difference is the activations' rounding alone.
TOL = {"float32": dict(atol=1e-5, rtol=1e-4), "bfloat16": dict(atol=2e-2, rtol=3e-2)}


class Loaded:
    def __init__(self, tmp, case, dtype):
        import pytorch_transformers_b200 as ptb
        name, overrides = CASES[case]
        self.name = name
        self.folder = tm.tiny_folder(str(tmp), name, bf16=(dtype == "bfloat16"), **overrides)
        self.model = ptb.AutoModelForCausalLM.from_pretrained(self.folder, dtype=dtype)
        self.cfg, self.w = plain.load_folder(self.folder, torch.float64)
        self.vocab = self.cfg["vocab_size"]

    def plain_logits(self, ids):
        return plain.model_logits(ids, self.cfg, self.w)


@pytest.fixture(scope="module")
def loaded(tmp_path_factory):
    cache = {}

    def get(case, dtype):
        if (case, dtype) not in cache:
            cache[(case, dtype)] = Loaded(tmp_path_factory.mktemp(f"{case}_{dtype}"), case, dtype)
        return cache[(case, dtype)]
    return get


def close(a, b, dtype, what=""):
    torch.testing.assert_close(a.double().cpu(), b.double().cpu(), msg=lambda m: f"{what}: {m}", **TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", sorted(CASES))
def test_each_request_alone_and_whole(loaded, case, dtype):
    L = loaded(case, dtype)
    cache = L.model.new_cache(256)
    for n, ids in zip((1, 5, 70, 129), tm.prompts(L.name, (1, 5, 70, 129), seed=11)):
        slot = cache.open()
        logits = L.model.step(cache, [slot], [ids], want="all")
        assert logits.shape == (n, L.vocab) and logits.dtype == torch.float32
        close(logits, L.plain_logits(ids), dtype, f"{case} whole prompt of {n}")
        cache.close(slot)
        cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B", "C", "D", "E", "F", "G"])
def test_last_32_tokens_one_by_one(loaded, case, dtype):
    L = loaded(case, dtype)
    cache = L.model.new_cache(192)
    for ids in tm.prompts(L.name, (33, 100, 140), seed=12):
        ref = L.plain_logits(ids)
        slot = cache.open()
        head = len(ids) - 32
        got = [L.model.step(cache, [slot], [ids[:head]], want="last")]
        for t in ids[head:]:
            got.append(L.model.step(cache, [slot], [[t]], want="last"))
        got = torch.cat(got)
        close(got, ref[head - 1:], dtype, f"{case} tail of {len(ids)}")
        cache.close(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B", "C", "D", "E", "F", "G"])
def test_batches_of_unequal_lengths_with_slot_reuse(loaded, case, dtype):
    L = loaded(case, dtype)
    # 9 requests, batches of 3, a cache that holds one batch only: pages and slots are reused
    lengths = [40, 7, 66, 1 + 12, 130, 64 + 3, 23, 65, 90]
    decode = [5, 3, 12, 12, 2, 9, 1, 20, 6]          # tokens fed one by one after the prompt part
    reqs = tm.prompts(L.name, lengths, seed=13)
    refs = [L.plain_logits(ids) for ids in reqs]
    cache = L.model.new_cache(64 * 6, max_slots=3)
    for b0 in range(0, 9, 3):
        idx = list(range(b0, b0 + 3))
        slots = {i: cache.open() for i in idx}
        assert sorted(slots.values()) == [0, 1, 2]
        heads = {i: lengths[i] - decode[i] for i in idx}
        out = L.model.step(cache, [slots[i] for i in idx], [reqs[i][:heads[i]] for i in idx], want="last")
        for r, i in enumerate(idx):
            close(out[r], refs[i][heads[i] - 1], dtype, f"{case} request {i} prompt end")
        live = list(idx)
        t = 0
        while live:
            done = [i for i in live if t >= decode[i]]
            for i in done:                              # shorter requests end earlier
                cache.close(slots[i])
            live = [i for i in live if i not in done]
            if not live:
                break
            out = L.model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + t]] for i in live], want="last")
            for r, i in enumerate(live):
                close(out[r], refs[i][heads[i] + t], dtype, f"{case} request {i} decode step {t}")
            t += 1
        cache.check()
        assert cache.live_tokens() == 0 and all(g.pool.in_use == 0 for g in cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_free_batch_equals_alone(loaded, dtype):
    # what else is in the batch changes nothing beyond rounding: in float32 not even that
    L = loaded("B", dtype)
    reqs = tm.prompts("B", (3, 50, 77), seed=14)
    cache = L.model.new_cache(512)
    alone = []
    for ids in reqs:
        s = cache.open()
        alone.append(L.model.step(cache, [s], [ids], want="all"))
        cache.close(s)
    slots = [cache.open() for _ in reqs]
    together = L.model.step(cache, slots, reqs, want="all")
    if dtype == "float32":
        assert torch.equal(together, torch.cat(alone))
    else:
        close(together, torch.cat(alone), dtype, "batch vs alone")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "C", "E"])
def test_long_decoding_and_first_tokens(loaded, case, dtype):
    L = loaded(case, dtype)
    ids = tm.prompts(L.name, (260,), seed=15)[0]
    ref = L.plain_logits(ids)
    cache = L.model.new_cache(320)
    slot = cache.open()
    got = [L.model.step(cache, [slot], [[t]], want="last") for t in ids]   # from the very first token on
    got = torch.cat(got)
    close(got[:4], ref[:4], dtype, f"{case} first tokens")
    close(got, ref, dtype, f"{case} 260 single-token steps")
    assert cache.length(slot) == 260


@pytest.mark.parametrize("case", ["A", "B", "C", "D"])
def test_greedy_generation_through_the_entry_point(loaded, case):
    L = loaded(case, "float32")
    prompts = tm.prompts(L.name, (5, 11, 17, 2), seed=16)
    out = L.model.generate(prompts, max_new_tokens=8, do_sample=False, eos_token_id=None, max_batch_size=3)
    for p, seq in zip(prompts, out):
        assert seq[:len(p)] == p
        assert seq[len(p):] == plain.greedy(p, L.cfg, L.w, 8)
    # the reference's calling form: left-padded ids with an attention mask
    width = max(len(p) for p in prompts)
    ids = torch.zeros(len(prompts), width, dtype=torch.long)
    mask = torch.zeros_like(ids)
    for i, p in enumerate(prompts):
        ids[i, width - len(p):] = torch.tensor(p)
        mask[i, width - len(p):] = 1
    seqs = L.model.generate(input_ids=ids, attention_mask=mask, max_new_tokens=8, do_sample=False,
                            eos_token_id=None)
    assert seqs.shape == (len(prompts), width + 8)
    for i, p in enumerate(prompts):
        assert seqs[i, width:].tolist() == out[i][len(p):]


def test_stop_tokens_end_a_sequence_early(loaded):
    L = loaded("B", "float32")
    prompts = tm.prompts("B", (9, 30, 4), seed=17)
    free = L.model.generate(prompts, max_new_tokens=10, eos_token_id=None)
    # make the 3rd new token of request 1 the stop token
    stop = free[1][len(prompts[1]) + 2]
    out = L.model.generate(prompts, max_new_tokens=10, eos_token_id=[stop], return_dict_in_generate=True)
    for i, p in enumerate(prompts):
        new_free = free[i][len(p):]
        want = new_free[:new_free.index(stop) + 1] if stop in new_free else new_free
        assert out.sequences[i][len(p):] == want
    assert out.finish_reasons[1] == "stop"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["E", "F"])
def test_decoding_across_a_bucket_of_pages_and_with_a_shrinking_batch(loaded, case, dtype):
    """Steps of single tokens are replayed as CUDA graphs keyed on the batch size and the width of
    the page tables (a multiple of 16 pages): decode from below 1024 tokens to above it, with
    three sequences of which two end early, and compare every step with the whole sequences."""
    L = loaded(case, dtype)
    assert L.model.use_graphs
    lengths = [1000, 1019, 40]
    decode = [40, 12, 30]
    reqs = tm.prompts(L.name, [n + d for n, d in zip(lengths, decode)], seed=18)
    refs = [L.plain_logits(ids) for ids in reqs]
    cache = L.model.new_cache(64 * 40)
    slots = [cache.open() for _ in reqs]
    out = L.model.step(cache, slots, [r[:n] for r, n in zip(reqs, lengths)], want="last")
    live = [0, 1, 2]
    for t in range(max(decode)):
        for row, i in enumerate(live):
            close(out[row], refs[i][lengths[i] + t - 1], dtype, f"{case} request {i} step {t}")
        live = [i for i in live if t < decode[i]]
        if not live:
            break
        out = L.model.step(cache, [slots[i] for i in live], [[reqs[i][lengths[i] + t]] for i in live], want="last")
    graphs = cache.__dict__.get("_step_graphs", {})
    assert len(graphs) >= 3          # batch sizes 3, 2, 1 and the wider page table
    # the same steps without graphs give the same numbers
    L.model.use_graphs = False
    try:
        cache2 = L.model.new_cache(64 * 20)
        s = cache2.open()
        L.model.step(cache2, [s], [reqs[2][:lengths[2]]], want="none")
        plain_step = L.model.step(cache2, [s], [[reqs[2][lengths[2]]]], want="last")
    finally:
        L.model.use_graphs = True
    cache3 = L.model.new_cache(64 * 20)
    s = cache3.open()
    L.model.step(cache3, [s], [reqs[2][:lengths[2]]], want="none")
    graph_step = L.model.step(cache3, [s], [[reqs[2][lengths[2]]]], want="last")
    assert torch.equal(plain_step, graph_step)


@pytest.mark.parametrize("dtype", DTYPES)
def test_falcon_7b_widths_two_layers(tmp_path, dtype):
    """The real widths of Falcon-7B (hidden 4544 = 71 heads of 64, one K/V head, fused projection
    of 4672 rows, feed-forward 18176) in a two-layer model with a small vocabulary: prompts in one
    step, then tokens one by one, against the plain implementation."""
    import pytorch_transformers_b200 as ptb
    cfg = tm.config_dict("A", hidden_size=4544, num_attention_heads=71, ffn_hidden_size=18176, vocab_size=1000,
                         max_position_embeddings=2048)
    rng = np.random.Generator(np.random.PCG64(77))
    weights = {}
    for name, shape in tm.tensor_shapes(cfg).items():
        w = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
        weights[name] = w + np.float32(1.0) if (name.endswith(".weight") and len(shape) == 1) else w
    folder = tm.write_model_folder(str(tmp_path / "wide"), cfg, weights, bf16=(dtype == "bfloat16"))
    model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    raw, w = plain.load_folder(folder, torch.float64)
    g = np.random.Generator(np.random.PCG64(5))
    reqs = [g.integers(0, 1000, size=n).tolist() for n in (150, 9)]
    refs = [plain.model_logits(ids, raw, w) for ids in reqs]
    cache = model.new_cache(512)
    slots = [cache.open() for _ in reqs]
    heads = [140, 3]
    out = model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], want="last")
    for t in range(6):
        for row, i in enumerate(range(2)):
            close(out[row], refs[i][heads[i] + t - 1], dtype, f"7B widths request {i} step {t}")
        out = model.step(cache, slots, [[reqs[i][heads[i] + t]] for i in range(2)], want="last")
    model.build.kernels.check_device_errors("cuda")
    if dtype != "bfloat16":
        return
    # A batch of more than 48 single tokens runs in one stream, and there the 71 heads of the one K/V
    # head are the rows of the tcgen05 decode kernel: the two requests again, among 48 copies of the
    # second one that start together, captured as a graph and
    # replayed, with a key page boundary inside the run.
    cache.close_all()
    cache = model.new_cache(64 * 60)
    K = model.build.kernels
    calls = []
    real = K.attention_decode_tc
    K.attention_decode_tc = lambda *a, **kw: (calls.append(a[0].shape[0]), real(*a, **kw))[1]
    try:
        many = [reqs[0], reqs[1]] + [reqs[1]] * 48
        starts = [60, 3] + [3] * 48
        slots = [cache.open() for _ in many]
        for i0 in range(0, len(many), 8):     # prompts a few at a time: 50 x 60 tokens would be one long step
            model.step(cache, slots[i0:i0 + 8], [r[:h] for r, h in zip(many[i0:i0 + 8], starts[i0:i0 + 8])], want="last")
        for t in range(6):
            out = model.step(cache, slots, [[many[i][starts[i] + t]] for i in range(len(many))], want="last")
            # What this part checks is the plumbing (pages, positions, rows, graph replay), whose faults
            # show as errors of the size of the logits (standard deviation 1.3 here). The elementwise
            # tolerance of the tests above sits at the rounding noise of bfloat16 at this width (measured
            # on whole prompts of this model: mean error 0.006, some of 150,000 elements at 1.4 times the
            # allowance), so the check here is on the error's mean and maximum; the kernel's own numerics
            # are pinned in the kernel tests.
            for r in (0, 1):
                err = (out[r].double().cpu() - refs[r][starts[r] + t]).abs()
                assert err.mean() < 0.01 and err.max() < 0.06, (r, t, float(err.mean()), float(err.max()))
            # the copies went through prompt steps of different sizes (other tiles of the library's matrix
            # products), so they agree to rounding, not bit for bit
            for r in (17, 39):
                err = (out[r].double().cpu() - refs[1][starts[1] + t]).abs()
                assert err.mean() < 0.01 and err.max() < 0.06, (r, t, float(err.mean()), float(err.max()))
    finally:
        K.attention_decode_tc = real
    assert calls and all(n == 50 for n in calls)
    K.check_device_errors("cuda")


@pytest.mark.parametrize("case", ["B", "E"])
def test_long_prompt_batches_are_fed_in_several_steps(loaded, case):
    L = loaded(case, "float32")
    prompts = tm.prompts(L.name, (70, 3, 41, 150, 9), seed=19)
    whole = L.model.generate(prompts, max_new_tokens=5, eos_token_id=None, return_dict_in_generate=True,
                             output_logits=True)
    for limit in (64, 100, 7):
        cut = L.model.generate(prompts, max_new_tokens=5, eos_token_id=None, max_step_tokens=limit,
                               return_dict_in_generate=True, output_logits=True)
        assert cut.sequences == whole.sequences
        for a, b in zip(cut.logits, whole.logits):
            torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("case", ["B", "E", "G"])
def test_prompts_through_the_tensor_memory_linear_layer(loaded, case, monkeypatch):
    """With the tcgen05 linear layer switched on for steps of 17 to 128 rows, prompts and batches of
    that size give the plain implementation's logits (the switch is off by default: the library
    product is faster)."""
    from pytorch_transformers_b200 import kernels as K
    from pytorch_transformers_b200.parts import linear as linear_mod
    calls = []
    real = K.tc_linear
    monkeypatch.setattr(K, "tc_linear", lambda *a, **kw: (calls.append(a[0].shape[0]), real(*a, **kw))[1])
    monkeypatch.setattr(linear_mod, "TC_LINEAR_ROWS", 128)
    L = loaded(case, "bfloat16")
    cache = L.model.new_cache(64 * 6)
    lengths = [70, 20, 31]
    reqs = tm.prompts(L.name, lengths, seed=21)
    slots = [cache.open() for _ in reqs]
    out = L.model.step(cache, slots, reqs, want="last")       # 121 rows in one step
    for r, ids in enumerate(reqs):
        close(out[r], L.plain_logits(ids)[-1], "bfloat16", f"{case} request {r}")
    K.check_device_errors(out.device)
    assert calls and all(16 < n <= 128 for n in calls)
    cache.close_all()
