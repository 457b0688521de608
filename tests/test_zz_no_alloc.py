"""The entry point that allocates nothing (csrc/no_alloc.h), called through its exported C symbol.

Some users of the kernel library cannot get device memory when they call it: they embed the C
interface with a fixed memory budget and no caching allocator, or they may not wait for the
driver's allocation lock. For them split decode attention exists in a form whose workspace is an array inside
the library. This test builds a decode batch with the package's own cache, runs the ordinary
entry point (workspace from the caller) and the fixed-workspace entry point on the same inputs,
twice in a row with different batches, and wants the same outputs; it also checks that a call
whose partial results would not fit is refused without a launch.

The file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _decode_inputs(K, pasts, heads, kv_heads, d, seed):
    """q for one new token per sequence and a cache that holds `pasts[b] + 1` keys and values."""
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.attention import AttentionTiles
    from pytorch_transformers_b200.parts.base import CacheNeed
    g = torch.Generator().manual_seed(seed)
    qpk = heads // kv_heads
    width = kv_heads * (qpk + 2) * d
    cache = Cache([(0, CacheNeed("full", kv_heads, d), None)], sum((p + 64) // 64 * 64 for p in pasts),
                  torch.bfloat16, "cuda")
    slots = [cache.open() for _ in pasts]
    k_pool, v_pool, gi = cache.entry_storage(0)
    ctx = StepContext(cache, slots, [[0] * p for p in pasts], 1, [[] for _ in pasts], [AttentionTiles(K)])
    fused = torch.randn(sum(pasts), width, generator=g).bfloat16().cuda()
    K.split_rotate_store(fused, k_pool, v_pool, ctx.batch_c[gi], None, kv_heads, qpk, d)
    ctx.commit()
    ctx = StepContext(cache, slots, [[0]] * len(pasts), 1, [[] for _ in pasts], [AttentionTiles(K)])
    fused = torch.randn(len(pasts), width, generator=g).bfloat16().cuda()
    q = K.split_rotate_store(fused, k_pool, v_pool, ctx.batch_c[gi], None, kv_heads, qpk, d)
    return q, k_pool, v_pool, ctx, gi, cache


def _tiles(ctx):
    return ctx.plan("attention_tiles")


def _call_fixed(lib, q, k_pool, v_pool, ctx, gi, kv_heads, hpk, warps, splits, watch_driver=False):
    """Call the exported symbol. With ``watch_driver`` the device's free memory as the driver counts it
    (cudaMemGetInfo: it sees a cudaMalloc by anybody in the process, which torch's own counter does not)
    must be the same after the call as before it. The first launch of a kernel may load its code, which
    takes device memory, so the watch is for calls after the first."""
    n, heads, d = q.shape
    out = torch.full((n, heads * d), float("nan"), dtype=q.dtype, device=q.device)
    torch.cuda.synchronize()
    held, free = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    fn = lib.ptb_attention_mma_fixed_scratch
    fn.restype = ctypes.c_int
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = fn(p(q), p(k_pool), p(v_pool), p(out), ctypes.byref(ctx.batch_c[gi]), p(_tiles(ctx).dev["mtile_seq"]),
            p(_tiles(ctx).dev["mtile_q0"]), _tiles(ctx).facts["n_mma_tiles"], ctypes.c_void_p(0), heads, kv_heads, d, hpk, 1, splits, warps,
            ctypes.c_float(1.0 / math.sqrt(d)), 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == held      # the call took nothing from torch's allocator
    if watch_driver:
        assert torch.cuda.mem_get_info()[0] == free   # nor from the driver
    return rc, out


def test_fixed_workspace_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from pytorch_transformers_b200 import kernels as K, native
    lib = native.library()
    K.lib()
    lib.ptb_attention_mma_fixed_scratch_strerror.restype = ctypes.c_char_p
    lib.ptb_attention_mma_fixed_scratch_capacity.restype = ctypes.c_longlong
    assert lib.ptb_attention_mma_fixed_scratch_capacity() == 4 * 1024 * 1024
    cases = [dict(pasts=[700, 63, 200, 1], heads=71, kv_heads=1, d=64, splits=5, seed=1),
             dict(pasts=[130, 900], heads=8, kv_heads=2, d=128, splits=3, seed=2)]
    for c in cases:
        q, k_pool, v_pool, ctx, gi, cache = _decode_inputs(K, c["pasts"], c["heads"], c["kv_heads"], c["d"], c["seed"])
        qpk = c["heads"] // c["kv_heads"]
        hpk, warps = qpk, (qpk + 15) // 16
        want = K.attention_mma(q, k_pool, v_pool, ctx.batch_c[gi], _tiles(ctx).dev["mtile_seq"], _tiles(ctx).dev["mtile_q0"],
                               _tiles(ctx).facts["n_mma_tiles"], None, c["kv_heads"], 1.0 / math.sqrt(c["d"]), 0, 1, hpk, warps,
                               c["splits"])
        for again in (False, True):        # the second call finds the first one's partial results in the array
            rc, got = _call_fixed(lib, q, k_pool, v_pool, ctx, gi, c["kv_heads"], hpk, warps, c["splits"],
                                  watch_driver=again)
            assert rc == 0, lib.ptb_attention_mma_fixed_scratch_strerror(rc)
            assert not torch.isnan(got.float()).any()
            torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
            assert torch.equal(got, want)      # same kernels, same order of sums
        del cache


def test_a_call_that_does_not_fit_is_refused_without_a_launch():
    from pytorch_transformers_b200 import kernels as K, native
    lib = native.library()
    K.lib()
    lib.ptb_attention_mma_fixed_scratch_strerror.restype = ctypes.c_char_p
    q, k_pool, v_pool, ctx, gi, cache = _decode_inputs(K, [100] * 40, 71, 1, 64, seed=3)
    # 40 tiles x 64 splits x 80 rows x 66 floats = 13.5 M floats > 4 Mi
    assert K.attention_mma_scratch_floats(40, 71, 1, 71, 64, 5, 64) > 4 * 1024 * 1024
    rc, out = _call_fixed(lib, q, k_pool, v_pool, ctx, gi, 1, 71, 5, 64, watch_driver=True)
    assert rc == 5
    assert b"16 MiB" in lib.ptb_attention_mma_fixed_scratch_strerror(rc)
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all()     # nothing was written
    # without splits no workspace is needed at all and the same call goes through
    rc, out = _call_fixed(lib, q, k_pool, v_pool, ctx, gi, 1, 71, 5, 1)
    assert rc == 0 and not torch.isnan(out.float()).any()
    # sizes that the kernel does not take are refused before the workspace is counted
    for bad in (dict(warps=9), dict(hpk=0), dict(splits=70000)):
        kw = dict(hpk=71, warps=5, splits=2)
        kw.update(bad)
        rc, out = _call_fixed(lib, q, k_pool, v_pool, ctx, gi, 1, kw["hpk"], kw["warps"], kw["splits"])
        assert rc == 2 and torch.isnan(out.float()).all()
