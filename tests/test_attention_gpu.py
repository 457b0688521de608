"""The split/rotate/store kernel and attention over the paged cache, alone, against plain attention
of whole sequences: head sizes in steps of 16 and one that is not, any number of heads and
groups, prompts, chunks after a past, single tokens, keys far back, page and window edges."""
import pytest
import torch

from engine_helpers import attention_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from pytorch_transformers_b200 import kernels
    kernels.lib()
    assert kernels.lib().ptb_attention_generic_tile_rows() == kernels.generic_tile_rows()
    return kernels


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


SHAPES = [  # heads, kv_heads, head_dim
    (4, 1, 16), (8, 2, 12), (6, 6, 16), (6, 3, 32), (71, 1, 64), (5, 5, 48), (4, 2, 128), (3, 1, 80), (2, 1, 256),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,d", SHAPES)
@pytest.mark.parametrize("position", ["rotary", "alibi"])
def test_prompts_of_unequal_lengths(K, dtype, heads, kv, d, position):
    out, ref = attention_case(K, dtype, heads, kv, d, pasts=[0, 0, 0, 0], news=[1, 17, 64, 131], position=position)
    torch.testing.assert_close(out, ref, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,d", [(4, 1, 16), (8, 2, 12), (71, 1, 64), (6, 3, 32)])
@pytest.mark.parametrize("position", ["rotary", "alibi"])
def test_single_tokens_and_chunks_after_a_past(K, dtype, heads, kv, d, position):
    # decode at a page's last slot, at a page's first slot, in the middle; a chunk across a page edge
    out, ref = attention_case(K, dtype, heads, kv, d, pasts=[63, 64, 200, 1, 60], news=[1, 1, 1, 1, 10],
                              position=position, seed=3)
    torch.testing.assert_close(out, ref, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("key_pos", [0, 63, 64, 300])
def test_a_far_key_among_hundreds_is_found(K, dtype, key_pos):
    out, ref = attention_case(K, dtype, 5, 1, 32, pasts=[0, 699], news=[40, 1], position="alibi" if key_pos % 2 else "none",
                              seed=5, needle=(1, key_pos))
    torch.testing.assert_close(out, ref, **tol(dtype))
    # the needle row really is dominated by one key: its output is far from the mean of values
    assert ref[-1].abs().max() > 0.5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [1, 5, 64, 65, 100])
def test_window(K, dtype, window):
    out, ref = attention_case(K, dtype, 4, 2, 16, pasts=[0, 130, 64], news=[150, 1, 3], position="rotary",
                              window=window, seed=7)
    torch.testing.assert_close(out, ref, **tol(dtype))


# ------------------------------------------------------------------------------ tensor-core kernel
MMA_SHAPES = [(71, 1, 64), (4, 1, 64), (8, 2, 64), (32, 8, 128), (128, 8, 64), (6, 6, 64), (5, 1, 128), (3, 3, 128)]
BF = torch.bfloat16


@pytest.mark.parametrize("heads,kv,d", MMA_SHAPES)
@pytest.mark.parametrize("position", ["rotary", "alibi"])
@pytest.mark.parametrize("splits", [1, 3])
def test_mma_single_tokens(K, heads, kv, d, position, splits):
    out, ref = attention_case(K, BF, heads, kv, d, pasts=[63, 64, 200, 1, 700, 127], news=[1] * 6,
                              position=position, seed=3, mma=(None, splits))
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("heads,kv,d", MMA_SHAPES)
@pytest.mark.parametrize("news", [[1, 17, 64, 131], [5, 16, 9], [40, 64, 1], [300]])
def test_mma_prompts(K, heads, kv, d, news):
    out, ref = attention_case(K, BF, heads, kv, d, pasts=[0] * len(news), news=news, position="rotary", seed=4,
                              mma=(None, 1))
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("news,pasts", [([10, 3], [60, 130]), ([70, 2], [1, 64]), ([129], [200])])
@pytest.mark.parametrize("hpk", [1, None])
def test_mma_chunks_after_a_past(K, news, pasts, hpk):
    out, ref = attention_case(K, BF, 8, 2, 64, pasts=pasts, news=news, position="alibi", seed=6, mma=(hpk, 1))
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("key_pos", [0, 63, 64, 300, 698])
def test_mma_far_key(K, key_pos):
    out, ref = attention_case(K, BF, 71, 1, 64, pasts=[0, 699], news=[1, 1], position="none", seed=5,
                              needle=(1, key_pos), mma=(None, 4))
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("window", [1, 5, 64, 65, 100])
@pytest.mark.parametrize("news,pasts,splits", [([150, 1, 3], [0, 130, 64], 1), ([1, 1, 1], [300, 5, 64], 2)])
def test_mma_window(K, window, news, pasts, splits):
    out, ref = attention_case(K, BF, 4, 2, 64, pasts=pasts, news=news, position="rotary", window=window, seed=7,
                              mma=(None, splits))
    torch.testing.assert_close(out, ref, **tol(BF))


def test_mma_refuses_what_it_does_not_take(K):
    from pytorch_transformers_b200.kernels import KernelError
    assert not K.attention_mma_supports(48) and K.attention_mma_supports(64) and K.attention_mma_supports(128)
    with pytest.raises(KernelError):
        attention_case(K, BF, 4, 1, 48, pasts=[0], news=[5], mma=(None, 1))
    with pytest.raises(KernelError):
        attention_case(K, torch.float32, 4, 1, 64, pasts=[0], news=[5], mma=(None, 1))


# ------------------------------------------------------------------------------ one-kernel decode
@pytest.mark.parametrize("heads,kv,d", MMA_SHAPES)
@pytest.mark.parametrize("position", ["rotary", "alibi"])
@pytest.mark.parametrize("splits", [1, 2, 3, 4, 7, 8])
def test_fused_decode(K, heads, kv, d, position, splits):
    # new tokens at a page's last slot, its first slot, in the middle, as the second token, far out
    out, ref = attention_case(K, BF, heads, kv, d, pasts=[63, 64, 200, 1, 700, 127], news=[1] * 6,
                              position=position, seed=3, fused_decode=(None, splits))
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("heads,kv,d", MMA_SHAPES)
@pytest.mark.parametrize("position", ["rotary", "alibi"])
@pytest.mark.parametrize("splits,key_split", [(1, 2), (1, 4), (3, 2), (5, 4), (8, 2)])
def test_fused_decode_keys_of_a_page_shared_among_warp_groups(K, heads, kv, d, position, splits, key_split):
    qpk = heads // kv
    if ((min(qpk, 128) + 15) // 16) * key_split > K.decode_max_warps(d):
        pytest.skip("more warps than a block of this kernel takes")
    out, ref = attention_case(K, BF, heads, kv, d, pasts=[63, 64, 200, 1, 700, 127], news=[1] * 6,
                              position=position, seed=3, fused_decode=(None, splits, key_split))
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("key_pos,key_split", [(0, 2), (64 + 17, 4), (698, 4), (699, 2)])
def test_fused_decode_far_key_with_key_groups(K, key_pos, key_split):
    out, ref = attention_case(K, BF, 8, 2, 64, pasts=[0 + 5, 699], news=[1, 1], position="none", seed=5,
                              needle=(1, key_pos), fused_decode=(None, 3, key_split))
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("window,key_split", [(1, 2), (5, 4), (65, 4), (100, 2)])
def test_fused_decode_window_with_key_groups(K, window, key_split):
    out, ref = attention_case(K, BF, 4, 2, 64, pasts=[300, 5, 64], news=[1, 1, 1], position="rotary", window=window,
                              seed=7, fused_decode=(None, 2, key_split))
    torch.testing.assert_close(out, ref, **tol(BF))


# ------------------------------------------------------------------------------ one-kernel decode on tcgen05
@pytest.mark.parametrize("heads,kv", [(71, 1), (128, 1), (33, 1), (80, 2), (132, 4)])
@pytest.mark.parametrize("position", ["rotary", "none"])
@pytest.mark.parametrize("splits", [1, 2, 3, 8])
def test_fused_decode_tc(K, heads, kv, position, splits):
    assert K.attention_decode_tc_supports(64, heads // kv)
    assert not K.attention_decode_tc_supports(64, 32) and not K.attention_decode_tc_supports(128, 64)
    assert not K.attention_decode_tc_supports(64, 129)
    # new tokens at a page's last slot, its first slot, in the middle, as the second token, far out
    out, ref = attention_case(K, BF, heads, kv, 64, pasts=[63, 64, 200, 1, 700, 127], news=[1] * 6,
                              position=position, seed=3, fused_decode=("tc", splits))
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("heads,kv", [(71, 1), (80, 2)])
@pytest.mark.parametrize("splits,teams", [(1, 2), (1, 5), (2, 3), (4, 4), (8, 2)])
def test_fused_decode_tc_teams_of_clusters(K, heads, kv, splits, teams):
    # several clusters share a sequence's pages and join through the workspace; sequences with fewer pages
    # than blocks leave some blocks without pages; launched twice, so the tickets must have been put back
    for seed in (3, 4):
        out, ref = attention_case(K, BF, heads, kv, 64, pasts=[63, 64, 200, 1, 1500, 127], news=[1] * 6,
                                  position="rotary", seed=seed, fused_decode=("tc", splits, teams))
        torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("key_pos", [0, 64, 1400, 1499])
def test_fused_decode_tc_teams_far_key_and_own_key(K, key_pos):
    out, ref = attention_case(K, BF, 71, 1, 64, pasts=[0 + 5, 1499], news=[1, 1], position="none", seed=5,
                              needle=(1, key_pos), fused_decode=("tc", 2, 4))
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("key_pos", [0, 64, 698, 699])
def test_fused_decode_tc_far_key_and_own_key(K, key_pos):
    out, ref = attention_case(K, BF, 71, 1, 64, pasts=[0 + 5, 699], news=[1, 1], position="none", seed=5,
                              needle=(1, key_pos), fused_decode=("tc", 4))
    torch.testing.assert_close(out, ref, **tol(BF))


def test_fused_decode_tc_repeated_steps(K):
    # three single-token steps in a row on the same cache: each step's key must be in the cache for the next
    for seed in (1, 2):
        out, ref = attention_case(K, BF, 71, 1, 64, pasts=[300, 65, 5], news=[1, 1, 1], position="rotary", seed=seed,
                                  fused_decode=("tc", 2))
        torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("hpk", [16, 32, None])
def test_fused_decode_head_chunks_and_repeated_launches(K, hpk):
    # 71 heads in chunks of 16 or 32: several blocks share a K/V head; launched twice so that the
    # tickets of the first launch must have been put back
    for seed in (1, 2):
        out, ref = attention_case(K, BF, 71, 1, 64, pasts=[300, 65, 5], news=[1, 1, 1], position="rotary", seed=seed,
                                  fused_decode=(hpk, 4))
        torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("heads,kv,d,hpk,key_split", [(71, 1, 64, None, 1), (71, 1, 64, 32, 1), (32, 8, 128, None, 4),
                                                      (8, 2, 64, None, 2), (128, 8, 64, None, 2)])
@pytest.mark.parametrize("splits,teams", [(1, 3), (2, 2), (4, 5), (8, 2)])
@pytest.mark.parametrize("position", ["rotary", "alibi"])
def test_fused_decode_teams_of_clusters(K, heads, kv, d, hpk, key_split, splits, teams, position):
    # several clusters share a sequence's pages and join through the workspace; short sequences leave
    # blocks without pages; launched twice, so the tickets must have been put back
    for seed in (3, 4):
        out, ref = attention_case(K, BF, heads, kv, d, pasts=[63, 64, 200, 1, 1500, 127], news=[1] * 6,
                                  position=position, seed=seed, fused_decode=(hpk, splits, key_split, teams))
        torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("key_pos", [0, 64, 1400, 1499])
def test_fused_decode_teams_far_key_and_own_key(K, key_pos):
    out, ref = attention_case(K, BF, 71, 1, 64, pasts=[0 + 5, 1499], news=[1, 1], position="none", seed=5,
                              needle=(1, key_pos), fused_decode=(None, 2, 1, 4))
    torch.testing.assert_close(out, ref, **tol(BF))


def test_fused_decode_teams_with_window(K):
    out, ref = attention_case(K, BF, 4, 2, 64, pasts=[900, 5, 64], news=[1, 1, 1], position="rotary", window=300,
                              seed=7, fused_decode=(None, 2, 2, 3))
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("key_pos", [0, 64, 698, 699])
def test_fused_decode_far_key_and_own_key(K, key_pos):
    out, ref = attention_case(K, BF, 71, 1, 64, pasts=[0 + 5, 699], news=[1, 1], position="none", seed=5,
                              needle=(1, key_pos), fused_decode=(None, 4))
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("window", [1, 5, 64, 65, 100])
def test_fused_decode_window(K, window):
    out, ref = attention_case(K, BF, 4, 2, 64, pasts=[300, 5, 64], news=[1, 1, 1], position="rotary", window=window,
                              seed=7, fused_decode=(None, 2))
    torch.testing.assert_close(out, ref, **tol(BF))


def test_rope_table_equals_in_kernel_angles(K):
    from engine_helpers import attention_case as case
    for dtype in (torch.float32, BF):
        a, ref = case(K, dtype, 4, 2, 64, pasts=[0, 3], news=[70, 9], position="rotary", seed=9)
        torch.testing.assert_close(a, ref, **tol(dtype))


# ------------------------------------------------------------------------------ tcgen05 prompt kernel
@pytest.mark.parametrize("heads,kv", [(1, 1), (3, 1), (71, 1), (8, 2), (4, 4), (2, 1), (12, 2)])
@pytest.mark.parametrize("news,pasts", [([128], [0]), ([65], [0]), ([129, 300, 70], [0, 0, 0]), ([200, 66], [130, 63]),
                                        ([1000], [0])])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("position", ["rotary", "alibi"])
def test_tc_prompts(K, heads, kv, news, pasts, d, position):
    assert K.lib().ptb_attention_tc_tile_tokens() == K.TC_TILE_TOKENS and K.attention_tc_supports(d)
    assert not K.attention_tc_supports(96) and not K.attention_tc_supports(256)
    out, ref = attention_case(K, BF, heads, kv, d, pasts=pasts, news=news, position=position, seed=11, tc=True)
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("heads,kv", [(2, 1), (3, 1), (8, 2), (12, 2), (5, 1)])
@pytest.mark.parametrize("news,pasts", [([128], [0]), ([65], [0]), ([129, 300, 70], [0, 0, 0]), ([200, 66], [130, 63]),
                                        ([1000], [0]), ([300], [200])])
@pytest.mark.parametrize("position", ["rotary", "alibi"])
def test_tc_prompts_two_heads_a_block(K, heads, kv, news, pasts, position):
    """Head size 128: two heads of a K/V group in one block, keys in steps of two pages (walks of an odd
    and an even number of pages, groups with an odd number of heads, whose last block has one chain)."""
    K.attention_tc_pairs(2)
    try:
        out, ref = attention_case(K, BF, heads, kv, 128, pasts=pasts, news=news, position=position, seed=12, tc=True)
    finally:
        K.attention_tc_pairs(1)
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("position", ["none", "alibi"])
def test_tc_far_key_two_heads_a_block(K, position):
    K.attention_tc_pairs(2)
    try:
        out, ref = attention_case(K, BF, 4, 2, 128, pasts=[0, 0], news=[70, 700], position=position, seed=5,
                                  needle=(1, 3), tc=True)
    finally:
        K.attention_tc_pairs(1)
    torch.testing.assert_close(out, ref, **tol(BF))


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("position", ["none", "alibi"])
def test_tc_far_key(K, d, position):
    out, ref = attention_case(K, BF, 2, 1, d, pasts=[0, 0], news=[70, 700], position=position, seed=5,
                              needle=(1, 3), tc=True)
    torch.testing.assert_close(out, ref, **tol(BF))


# ------------------------------------------------------------------------------ the same launch again and again
def _cache_with(K, kv, d, lengths, new):
    """A cache of one entry whose sequences hold `lengths` tokens of random keys and values, and the
    step that brings `new` tokens to each of them."""
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.attention import AttentionTiles
    from pytorch_transformers_b200.parts.base import CacheNeed
    cache = Cache([(0, CacheNeed("full", kv, d, 0), None)], sum(t + new + 64 for t in lengths), BF, "cuda")
    slots = [cache.open() for _ in lengths]
    for slot, t in zip(slots, lengths):
        if t:
            cache.reserve(slot, t)
            cache.commit(slot, t)
    ctx = StepContext(cache, slots, [[0] * new] * len(lengths), 1, [[]] * len(lengths), (AttentionTiles(K),))
    k_pool, v_pool, group = cache.entry_storage(0)
    gen = torch.Generator(device="cuda").manual_seed(3)
    k_pool.normal_(generator=gen)
    v_pool.normal_(generator=gen)
    return ctx, k_pool, v_pool, ctx.batch_c[group], gen


@pytest.mark.parametrize("heads,kv,d,tokens", [(71, 1, 64, 2048), (32, 8, 128, 1500), (12, 3, 128, 700)])
def test_tc_prompts_the_same_bits_every_time(K, heads, kv, d, tokens):
    """The roles of the prompt kernel meet at barriers only, and its warps run pages apart: a wait that
    takes one phase for another shows as a result that changes from launch to launch (it did, with a
    single row or a warp of rows off in their last page), long before it shows against the plain
    attention of a small case. Forty launches of the same work must give the same bits."""
    ctx, k_pool, v_pool, batch, gen = _cache_with(K, kv, d, [0, 130], tokens)
    tiles = ctx.plan("attention_tiles")
    K.attention_tc_pairs(2)       # head size 128: two heads a block also where the pairs do not fill the device
    q = torch.randn(2 * tokens, heads, d, device="cuda", generator=gen).to(BF)
    run = lambda: K.attention_tc(q, k_pool, v_pool, batch, tiles.dev["mtile_seq"], tiles.dev["mtile_q0"],
                                 tiles.facts["n_mma_tiles"], kv, d ** -0.5, None)
    try:
        first = run()
        for _ in range(40):
            assert torch.equal(run(), first)
    finally:
        K.attention_tc_pairs(1)
    K.check_device_errors("cuda")
    # and they are the right bits: the general kernel on the same tiles
    ref = K.attention_generic(q, k_pool, v_pool, batch, tiles.dev["tile_seq"], tiles.dev["tile_q0"],
                              tiles.facts["n_tiles"], None, kv, d ** -0.5, 0)
    torch.testing.assert_close(first.float(), ref.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("splits,teams", [(4, 1), (8, 1), (8, 4)])
def test_fused_decode_tc_the_same_bits_every_time(K, splits, teams):
    heads, kv, d = 71, 1, 64
    ctx, k_pool, v_pool, batch, gen = _cache_with(K, kv, d, [2048, 5000, 300, 1777], 1)
    fused = torch.randn(4, kv * (heads // kv + 2) * d, device="cuda", generator=gen).to(BF)
    inv = (1.0 / (10000 ** (torch.arange(0, d, 2).float() / d))).cuda()
    rope = K.rope_table(ctx.dev["tok_pos"], inv)
    run = lambda: K.attention_decode_tc(fused, k_pool, v_pool, batch, rope, kv, heads // kv, d, d ** -0.5, splits,
                                        n_teams=teams)
    first = run()
    for _ in range(40):
        assert torch.equal(run(), first)
    K.check_device_errors("cuda")


# ------------------------------------------------------------------------------ random shapes
@pytest.mark.parametrize("first_seed", range(0, 80, 20))
def test_tensor_core_kernels_on_random_shapes(K, first_seed):
    """The four tensor-core attention kernels on drawn head counts, groups, lengths, pasts and divisions of
    the pages (blocks a cluster, clusters a sequence, warp groups a page), against the plain attention. A
    division that a kernel refuses is a refusal with its error, never a wrong result."""
    import random
    from pytorch_transformers_b200.kernels import KernelError
    for seed in range(first_seed, first_seed + 20):
        r = random.Random(seed)
        kind = r.choice(["prompt", "prompt, two heads a block", "decode tcgen05", "decode mma"])
        try:
            if kind.startswith("prompt"):
                pair = kind != "prompt"
                d = 128 if pair else r.choice([64, 128])
                kv, qpk = r.choice([1, 2, 3]), (r.choice([2, 3, 4, 5]) if pair else r.choice([1, 2, 3, 4, 7]))
                n = r.choice([1, 2, 3])
                news = [r.randint(65, r.choice([130, 400, 900])) for _ in range(n)]
                pasts = [r.choice([0, 0, r.randint(65, 300)]) for _ in range(n)]
                if any(pasts) and not all(pasts):
                    pasts = [max(p, 70) for p in pasts]
                K.attention_tc_pairs(2 if pair else r.choice([0, 1]))
                try:
                    out, ref = attention_case(K, BF, kv * qpk, kv, d, pasts=pasts, news=news,
                                              position=r.choice(["rotary", "alibi"]), seed=seed, tc=True)
                finally:
                    K.attention_tc_pairs(1)
            elif kind == "decode tcgen05":
                kv, qpk, n = r.choice([1, 2]), r.choice([33, 40, 71, 100, 128]), r.choice([1, 2, 4])
                pasts = [r.randint(1, r.choice([100, 700, 2500])) for _ in range(n)]
                out, ref = attention_case(K, BF, kv * qpk, kv, 64, pasts=pasts, news=[1] * n,
                                          position=r.choice(["rotary", "none"]), seed=seed,
                                          fused_decode=("tc", r.choice([1, 2, 3, 4, 8]), r.choice([1, 1, 2, 3])))
            else:
                kv, qpk, d = r.choice([1, 2, 3, 8]), r.choice([1, 2, 4, 5, 16, 71]), r.choice([16, 32, 64, 128])
                qpk = 4 if kv * qpk > 142 else qpk
                n = r.choice([1, 2, 4])
                pasts = [r.randint(1, r.choice([100, 700, 2000])) for _ in range(n)]
                groups = r.choice([1, 1, 2, 4])
                if (min(qpk, 128) + 15) // 16 * groups > K.decode_max_warps(d):
                    groups = 1
                out, ref = attention_case(K, BF, kv * qpk, kv, d, pasts=pasts, news=[1] * n,
                                          position=r.choice(["rotary", "alibi"]), seed=seed,
                                          fused_decode=(None, r.choice([1, 2, 3, 4, 8]), groups, r.choice([1, 1, 2, 3])))
        except KernelError as refusal:
            assert "does not take" in str(refusal) or "too many" in str(refusal), (seed, kind, refusal)
            continue
        torch.testing.assert_close(out, ref, msg=lambda m: f"seed {seed} {kind}: {m}", **tol(BF))
