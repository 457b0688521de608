"""Decisions that shape a step of single tokens, checked without a GPU: how many blocks share a
sequence's pages, how many warp groups share a page's keys, when the mixer runs on a second
stream, which plan a mixer adds to a step. The thresholds behind them are measured on the device
and may be retuned; what is checked here is what must hold for any thresholds: no block without
pages, no launch beyond what the kernels take, rules that are monotone in the size of the work,
and a model that asks its own parts instead of carrying their numbers."""
from types import SimpleNamespace

import pytest
import torch

import tiny_models as tm

import pytorch_transformers_b200 as ptb
from pytorch_transformers_b200 import kernels
from pytorch_transformers_b200.engine.batch import StepContext, StepError
from pytorch_transformers_b200.parts import BuildContext, Part, PartSpec, make_part
from pytorch_transformers_b200.parts.attention import AttentionTiles

SMS = kernels.sm_count("cpu")          # without a device: the B200's count
SHAPES = ((71, 1, 64), (32, 8, 128), (128, 8, 64), (48, 1, 128), (40, 1, 64), (8, 2, 64), (6, 6, 64))


def attention(heads, kv_heads, head_dim, window=0, dtype=torch.bfloat16):
    build = BuildContext(torch.device("cpu"), dtype, kernels)
    return make_part(build, PartSpec("mixer", "attention", {"hidden": heads * head_dim, "heads": heads,
                                                            "kv_heads": kv_heads, "head_dim": head_dim,
                                                            "window": window}))


def decode_ctx(n_seqs, pages, context=None):
    context = context if context is not None else pages * 64 - 1
    return SimpleNamespace(n_seqs=n_seqs, pages_hint=pages, past=[context] * n_seqs, new=[1] * n_seqs,
                           n_tokens=n_seqs, side_stream=None)


@pytest.mark.parametrize("heads,kv,d", SHAPES)
def test_blocks_that_share_a_sequence(heads, kv, d):
    part = attention(heads, kv, d)
    hpk = min(heads // kv, 128)
    chunks = (heads // kv + hpk - 1) // hpk
    last = None
    for n_seqs in (1, 2, 8, 13, 64, 200, 1000):
        for pages in (1, 2, 3, 4, 9, 33, 129, 257):
            ctx = decode_ctx(n_seqs, pages)
            want = part._decode_splits(ctx, hpk)
            assert want >= 1
            if want > 1:
                assert want * 2 <= pages                              # every block has two pages or more
                assert want * n_seqs * kv * chunks <= 2 * SMS         # and the launch is two blocks an SM at most
            splits = max(s for s in kernels.DECODE_SPLITS if s <= want)
            teams = part._decode_teams(ctx, want, 4)
            assert teams >= 1
            if teams > 1:
                assert splits == max(kernels.DECODE_SPLITS)           # more clusters only when one is full
                assert teams * splits * 4 <= pages + 4 * splits       # four pages a block, give or take a cluster
                assert n_seqs * kv * chunks * splits * teams <= 2 * SMS + splits * n_seqs * kv * chunks
        # more sequences never get more blocks each
        w = part._decode_splits(decode_ctx(n_seqs, 257), hpk)
        assert last is None or w <= last
        last = w
    # a short context is not divided at all, whatever the batch
    assert part._decode_splits(decode_ctx(1, 2), hpk) == 1
    assert part._decode_splits(decode_ctx(1, 3), hpk) == 1


def test_a_window_bounds_the_pages_that_count():
    windowed = attention(8, 2, 64, window=100)
    full = attention(8, 2, 64)
    ctx = decode_ctx(1, 500)
    assert windowed._decode_pages(ctx) <= 100 // 64 + 2 < full._decode_pages(ctx)
    assert windowed._decode_splits(ctx, 4) <= max(1, windowed._decode_pages(ctx) // 2)
    assert windowed._decode_splits(ctx, 4) < full._decode_splits(ctx, 4)


@pytest.mark.parametrize("heads,kv,d", SHAPES)
def test_warp_groups_per_page_fit_the_block(heads, kv, d):
    part = attention(heads, kv, d)
    row_warps = (min(heads // kv, 128) + 15) // 16
    groups = part._decode_key_split(row_warps)
    assert groups in kernels.DECODE_KEY_SPLITS
    assert row_warps * groups <= kernels.decode_max_warps(d)
    # few warps of rows are what the groups are for: never fewer groups for fewer warps
    if row_warps > 1:
        assert part._decode_key_split(row_warps - 1) >= groups


def test_the_mixer_decides_about_the_second_stream_and_the_rule_is_monotone():
    for heads, kv, d in SHAPES:
        part = attention(heads, kv, d)
        flips = 0
        before = True
        for context in (64, 512, 2048, 8192, 16384, 65536, 1 << 20):
            now = part.runs_beside(decode_ctx(8, 0, context=context))
            flips += now != before
            assert not (now and not before)            # once the keys are too many, more keys never fit again
            before = now
        assert part.runs_beside(decode_ctx(1, 0, context=64))          # a tiny read always hides
        assert not part.runs_beside(decode_ctx(64, 0, context=1 << 20))
        assert flips == 1
        # the same bytes with wider heads fit no longer than with narrow ones
        assert kernels.decode_attention_fits_beside(1 << 20, 64) and kernels.decode_attention_fits_beside(1 << 20, 128)
        for b in (1 << 20, 30 << 20, 50 << 20):
            assert kernels.decode_attention_fits_beside(b, 64) or not kernels.decode_attention_fits_beside(b, 128)
    # a window bounds what a layer reads
    assert attention(8, 2, 64, window=1024).runs_beside(decode_ctx(8, 0, context=1 << 20))
    # the 32-bit path is for checking, one stream
    assert not attention(8, 2, 64, dtype=torch.float32).runs_beside(decode_ctx(1, 0, context=64))


def test_the_model_asks_its_mixers():
    cfg = ptb.FalconConfig.from_dict(tm.config_dict("E"))
    model = ptb.AutoModelForCausalLM.from_config(cfg, seed=0, dtype="bfloat16", device="cpu")
    model.device = torch.device("cuda")                 # the rule itself needs no device
    ctx = decode_ctx(8, 0, context=2048)
    assert model._two_streams(ctx)
    asked = []
    for m in model._mixers:
        m.runs_beside = lambda c, m=m: (asked.append(m), False)[1]
    assert not model._two_streams(ctx) and asked         # one mixer that declines is enough
    for m in model._mixers:
        del m.runs_beside
    assert not model._two_streams(decode_ctx(kernels.WEIGHT_STREAM_MAX_ROWS + 1, 0, context=64))
    assert Part.runs_beside(model._mixers[0], ctx) is False          # a mixer that says nothing stays on one stream


def test_a_mixers_plan_travels_with_the_step():
    cfg = ptb.FalconConfig.from_dict(tm.config_dict("A"))
    model = ptb.AutoModelForCausalLM.from_config(cfg, seed=0, dtype="float32", device="cpu")
    assert [p.plan_key for p in model.planners] == ["attention_tiles"]      # one plan for all attention layers
    cache = model.new_cache(64 * 8)
    slots = [cache.open() for _ in range(3)]
    ctx = StepContext(cache, slots, [[1] * 70, [2] * 5, [3] * 17], 512, [[0], [], [16]], model.planners)
    tiles = ctx.plan("attention_tiles")
    rows = kernels.generic_tile_rows()
    assert tiles.facts["n_tiles"] == sum(-(-n // rows) for n in (70, 5, 17))
    assert tiles.facts["mma_tokens"] == kernels.TC_TILE_TOKENS and tiles.facts["n_mma_tiles"] == 3
    # tiles by falling count of keys before them (their blocks start in this order, the longest walks first)
    assert tiles.dev["tile_seq"].tolist() == [0, 0, 0, 0, 2, 0, 1, 2]
    assert tiles.dev["tile_q0"].tolist() == [64, 48, 32, 16, 16, 0, 0, 0]
    assert sorted(zip(tiles.dev["tile_seq"].tolist(), tiles.dev["tile_q0"].tolist())) == \
        [(0, 0), (0, 16), (0, 32), (0, 48), (0, 64), (1, 0), (2, 0), (2, 16)]
    # a step of single tokens: one token a tile; the plan's numbers are part of the step's layout
    cache.close_all()
    slots = [cache.open() for _ in range(2)]
    one = StepContext(cache, slots, [[1], [2]], 512, [[0], [0]], model.planners)
    assert one.plan("attention_tiles").facts["mma_tokens"] == 1
    assert one.layout_key != ctx.layout_key and "attention_tiles" in str(one.layout_key)
    # a step that was built without a plan says which one is missing
    bare = StepContext(cache, slots, [[1], [2]], 512, [[0], [0]])
    with pytest.raises(StepError, match="attention_tiles"):
        bare.plan("attention_tiles")


def test_tile_sizes_come_from_the_kernels():
    class FakeKernels:
        TC_TILE_TOKENS = 256

        @staticmethod
        def generic_tile_rows():
            return 8

    ctx = SimpleNamespace(new=[100, 3], past=[0, 0],
                          tiles=lambda rows: ([0] * -(-100 // rows) + [1], list(range(0, 100, rows)) + [0]))
    plan = AttentionTiles(FakeKernels).plan(ctx)
    assert plan.facts == {"n_tiles": 14, "mma_tokens": 256, "n_mma_tiles": 2}


def test_rows_that_go_to_the_weight_streaming_kernel():
    # only what the kernel takes is ever preferred, and never more rows for the tall matrices than for the others
    for rows in range(1, 40):
        for k, n in ((4544, 4672), (4544, 65024), (8192, 32768), (4544 + 8, 4672)):
            if kernels.skinny_linear_preferred(rows, k, n):
                assert kernels.skinny_linear_takes(rows, k)
                assert rows == 1 or kernels.skinny_linear_preferred(rows - 1, k, n)
            if kernels.skinny_linear_preferred(rows, 4544, 65024):
                assert kernels.skinny_linear_preferred(rows, 4544, 4672)
    assert kernels.skinny_linear_preferred(1, 4544, 4672) and not kernels.skinny_linear_preferred(1, 4544 + 8, 4672)


def test_activation_names_match_the_kernels_table():
    import os
    import re
    src = open(os.path.join(os.path.dirname(kernels.__file__), "csrc", "common.cuh")).read()
    codes = {m.group(1): int(m.group(2)) for m in re.finditer(r"PTB_ACT_(\w+) = (\d+)", src)}
    assert codes.pop("COUNT") == len(codes) == len(set(kernels.ACTIVATIONS.values()))
    assert sorted(codes.values()) == sorted(set(kernels.ACTIVATIONS.values()))
    assert kernels.ACTIVATIONS["none"] == codes["NONE"] and kernels.ACTIVATIONS["gelu"] == codes["GELU_ERF"]
    assert kernels.ACTIVATIONS["gelu_new"] == kernels.ACTIVATIONS["gelu_pytorch_tanh"] == codes["GELU_TANH"]
    assert kernels.ACTIVATIONS["relu"] == codes["RELU"]
    # the switch lives in one place
    for name in os.listdir(os.path.join(os.path.dirname(kernels.__file__), "csrc")):
        if name.endswith(".cu"):
            assert "erff(" not in open(os.path.join(os.path.dirname(kernels.__file__), "csrc", name)).read(), name
