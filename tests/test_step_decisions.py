"""Decisions that shape a step of single tokens, checked without a GPU: how many blocks share a
sequence's pages, how many warp groups share a page's keys, and when the mixer runs on a second
stream. The numbers they rest on are measured on the device; these tests pin the rules."""
from types import SimpleNamespace

import torch

from pytorch_transformers_b200 import kernels
from pytorch_transformers_b200.engine.model import CausalLM
from pytorch_transformers_b200.parts import BuildContext, PartSpec, make_part


def attention(heads, kv_heads, head_dim, window=0):
    build = BuildContext(torch.device("cpu"), torch.bfloat16, kernels)
    return make_part(build, PartSpec("mixer", "attention", {"hidden": heads * head_dim, "heads": heads,
                                                            "kv_heads": kv_heads, "head_dim": head_dim,
                                                            "window": window}))


def test_blocks_per_sequence_fill_the_device_once():
    falcon_7b = attention(71, 1, 64)
    ctx = SimpleNamespace(n_seqs=8, pages_hint=33)
    assert falcon_7b._decode_splits(ctx, 71) == 16          # capped by two pages per block; the kernel takes 8
    assert max(s for s in kernels.DECODE_SPLITS if s <= 16) == 8
    ctx = SimpleNamespace(n_seqs=64, pages_hint=33)
    assert falcon_7b._decode_splits(ctx, 71) == 4           # 64 x 4 blocks: no second wave on 148 SMs
    ctx = SimpleNamespace(n_seqs=200, pages_hint=33)
    assert falcon_7b._decode_splits(ctx, 71) == 1
    ctx = SimpleNamespace(n_seqs=8, pages_hint=2)
    assert falcon_7b._decode_splits(ctx, 71) == 1           # a short context is not divided
    falcon_11b = attention(32, 8, 128)
    assert falcon_11b._decode_splits(SimpleNamespace(n_seqs=8, pages_hint=33), 4) == 4
    windowed = attention(8, 2, 64, window=100)
    assert windowed._decode_splits(SimpleNamespace(n_seqs=1, pages_hint=500), 4) == 1   # 100 keys: three pages


def test_warp_groups_per_page():
    assert attention(71, 1, 64)._decode_key_split(5) == 1      # five warps of rows already
    assert attention(32, 8, 128)._decode_key_split(1) == 4     # one warp of rows, head size 128
    assert attention(128, 8, 64)._decode_key_split(1) == 2     # one warp of rows, head size 64
    assert attention(64, 2, 128)._decode_key_split(2) == 4     # 2 x 4 = 8 warps, the most a block of size 128 takes
    for heads, kv, d in ((71, 1, 64), (32, 8, 128), (128, 8, 64), (48, 1, 128), (40, 1, 64)):
        part = attention(heads, kv, d)
        row_warps = (min(heads // kv, 128) + 15) // 16
        groups = part._decode_key_split(row_warps)
        assert groups in kernels.DECODE_KEY_SPLITS and row_warps * groups <= kernels.decode_max_warps(d)


def fake_step(batch, context, kv_heads, head_dim, tokens_per_seq=1, window=0):
    group = SimpleNamespace(need=SimpleNamespace(kv_heads=kv_heads, head_dim=head_dim, window=window),
                            k=torch.empty(0, dtype=torch.bfloat16))
    return SimpleNamespace(n_tokens=batch * tokens_per_seq, past=[context] * batch, new=[tokens_per_seq] * batch,
                           cache=SimpleNamespace(groups=[group]))


def test_second_stream_only_while_the_layers_key_value_read_is_small():
    model = SimpleNamespace(device=torch.device("cuda"), dtype=torch.bfloat16,
                            TWO_STREAM_MAX_TOKENS=CausalLM.TWO_STREAM_MAX_TOKENS,
                            TWO_STREAM_MAX_KV_BYTES=CausalLM.TWO_STREAM_MAX_KV_BYTES,
                            TWO_STREAM_MAX_KV_BYTES_WIDE_HEADS=CausalLM.TWO_STREAM_MAX_KV_BYTES_WIDE_HEADS)
    rule = lambda ctx: CausalLM._two_streams(model, ctx)
    assert rule(fake_step(8, 2048, 1, 64))            # Falcon-7B, batch 8: 4 MB a layer
    assert rule(fake_step(32, 2048, 1, 64))           # batch 32: 17 MB
    assert rule(fake_step(48, 2048, 1, 64))           # batch 48: 25 MB
    assert not rule(fake_step(64, 2048, 1, 64))       # more than 48 tokens
    assert not rule(fake_step(8, 2048, 8, 128))       # Falcon-11B, batch 8: 67 MB
    assert rule(fake_step(1, 2048, 8, 128))           # batch 1: 8 MB
    assert rule(fake_step(8, 2048, 8, 64))            # Falcon-40B, batch 8: 34 MB
    assert rule(fake_step(8, 16384, 1, 64))           # Falcon-7B, batch 8 at 16,384 keys: 34 MB
    assert not rule(fake_step(10, 16384, 1, 64))      # 42 MB
    assert not rule(fake_step(4, 2048, 8, 128))       # Falcon-11B, batch 4: 34 MB, but heads of size 128
    assert rule(fake_step(2, 2048, 8, 128))           # 17 MB
    assert rule(fake_step(8, 100000, 8, 64, window=1024))   # a window bounds what a layer reads
    assert not rule(fake_step(2, 10, 1, 64, tokens_per_seq=40))
    model.dtype = torch.float32
    assert not rule(fake_step(8, 2048, 1, 64))


def test_teams_of_clusters_for_long_sequences_in_small_batches():
    falcon_7b = attention(71, 1, 64)
    def teams(n_seqs, pages):
        ctx = SimpleNamespace(n_seqs=n_seqs, pages_hint=pages)
        return falcon_7b._decode_teams(ctx, falcon_7b._decode_splits(ctx, 71), 4)
    assert teams(8, 33) == 1         # 2,048 keys: one cluster of 8 blocks, four pages each
    assert teams(64, 33) == 1
    assert teams(8, 257) == 4        # 16,384 keys, batch 8: 8 x 32 blocks fill the device once
    assert teams(1, 257) == 8        # batch 1: four pages a block at least
    assert teams(1, 129) == 4
    assert teams(64, 257) == 1       # a large batch fills the device by itself


def test_rows_that_go_to_the_skinny_linear_kernel():
    assert kernels.skinny_linear_preferred(8, 4544, 4672)
    assert kernels.skinny_linear_preferred(12, 4544, 18176)
    assert not kernels.skinny_linear_preferred(13, 4544, 18176)       # the library from 13 rows on
    assert kernels.skinny_linear_preferred(4, 4544, 65024)            # the head: up to 4 rows
    assert not kernels.skinny_linear_preferred(8, 4544, 65024)
    assert not kernels.skinny_linear_preferred(8, 4544 + 8, 4672)     # K must be a multiple of 32
