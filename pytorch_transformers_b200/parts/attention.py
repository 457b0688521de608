"""The attention mixer: fused query/key/value projection, position encoding, attention over
the paged cache, output projection.

The fused projection's rows are grouped per K/V head as (q_per_kv query heads, K, V). This one
layout covers the three that the reference's ``_split_heads`` distinguishes
(src/transformers/models/falcon/modeling_falcon.py:269-298): the new decoder architecture
(kv_heads groups), multi-query (one group: all queries, K, V) and per-head q,k,v (heads
groups of one query). Query head h reads K/V head h // q_per_kv. Scores are
``(q.k + bias) / sqrt(head_dim)`` over the keys at positions <= the query's
(modeling_falcon.py:388-393, 1139-1144), softmax in float32.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

from .base import BuildContext, CacheNeed, ParamDecl, Part, PartSpec, register_part
from .linear import linear


MAX_HEAD_DIM = 256   # csrc/attention_generic.cu keeps a row's accumulators in registers up to this size


class AttentionTiles:
    """The attention kernels' view of a step, as a planner (engine.batch.StepPlan): the tiles of the
    general kernel ((sequence, first token) every ``generic_tile_rows`` tokens) and the tiles of the
    tensor-core kernels, which hold one token when every sequence brings a single token (all heads of a
    K/V group share the tile), else 16, 64 or the tcgen05 kernel's 128 tokens by the longest sequence.
    Tiles are listed by falling count of the keys that their first token sees: a tile's block walks
    that many keys and blocks start in the order of the list, so the long walks start first and the
    short ones fill the device's last wave instead of one long walk ending alone.
    All attention layers of a model share the one plan."""
    plan_key = "attention_tiles"

    @staticmethod
    def _longest_first(ctx, seqs, firsts):
        order = sorted(range(len(seqs)), key=lambda i: -(ctx.past[seqs[i]] + firsts[i]))   # stable: ties keep their order
        return [seqs[i] for i in order], [firsts[i] for i in order]

    def __init__(self, kernels):
        self.kernels = kernels

    def plan(self, ctx):
        from ..engine.batch import StepPlan
        k = self.kernels
        longest = max(ctx.new)
        sizes = (16, 64, k.TC_TILE_TOKENS)
        mma_tokens = 1 if longest == 1 else next((t for t in sizes if longest <= t), sizes[-1])
        tile_seq, tile_q0 = self._longest_first(ctx, *ctx.tiles(k.generic_tile_rows()))
        mtile_seq, mtile_q0 = self._longest_first(ctx, *ctx.tiles(mma_tokens))
        return StepPlan(arrays={"tile_seq": tile_seq, "tile_q0": tile_q0, "mtile_seq": mtile_seq, "mtile_q0": mtile_q0},
                        facts={"n_tiles": len(tile_seq), "mma_tokens": mma_tokens, "n_mma_tiles": len(mtile_seq)})


@register_part("mixer", "attention")
class Attention(Part):
    graph_safe = True
    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, heads: int, kv_heads: int, head_dim: int,
                 bias: bool = False, window: int = 0, scale: Optional[float] = None):
        super().__init__(build, spec)
        if heads % kv_heads:
            raise ValueError(f"heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        if not (0 < head_dim <= MAX_HEAD_DIM):
            raise ValueError(f"the attention kernels take head sizes from 1 to {MAX_HEAD_DIM}, got {head_dim}")
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        self.q_per_kv = self.heads // self.kv_heads
        self.has_bias, self.window = bool(bias), int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = self.children.get("position")
        self.p_qkv_weight = self.p_qkv_bias = self.p_out_weight = self.p_out_bias = None
        import torch
        self._bf16 = torch.bfloat16

    def param_decls(self) -> Dict[str, ParamDecl]:
        fused = (self.heads + 2 * self.kv_heads) * self.head_dim
        d = {"qkv.weight": ParamDecl((fused, self.hidden)),
             "out.weight": ParamDecl((self.hidden, self.heads * self.head_dim))}
        if self.has_bias:
            d["qkv.bias"] = ParamDecl((fused,), role="vector")
            d["out.bias"] = ParamDecl((self.hidden,), role="vector")
        return d

    def cache_need(self):
        return CacheNeed("window" if self.window > 0 else "full", self.kv_heads, self.head_dim, self.window)

    def state_need(self):
        return None

    def planner(self):
        return AttentionTiles(self.build.kernels)

    def runs_beside(self, ctx) -> bool:
        """On a second stream while the keys and values that this layer reads in the step are few beside
        the feed-forward's weights (the limits are the kernels': kernels.decode_attention_fits_beside)."""
        import torch
        if self.build.dtype != torch.bfloat16:
            return False
        lengths = (p + n for p, n in zip(ctx.past, ctx.new))
        keys = sum(min(t, self.window) if self.window else t for t in lengths)
        return self.build.kernels.decode_attention_fits_beside(keys * self.kv_heads * self.head_dim * 2 * 2, self.head_dim)

    fuses_add = True

    def forward(self, x, ctx, entry, add=None):
        """Attention of ``x`` (already normed); ``add`` [tokens, hidden] is summed into the result in
        the output projection's float32 epilogue."""
        k = self.build.kernels
        fused = linear(k, x, self.p_qkv_weight, self.p_qkv_bias)
        k_pool, v_pool, group = ctx.cache.entry_storage(entry.cache_entry)
        batch = ctx.batch_c[group]
        rope = ctx.rope(self.position)
        slopes = self.position.score_bias() if self.position is not None else None
        inter = bool(getattr(self.position, "interleaved", False))   # rotated pairs (2 i, 2 i + 1) instead of (i, i + n)
        tiles = ctx.plan(AttentionTiles.plan_key)
        if tiles.facts["mma_tokens"] == 1 and fused.dtype == self._bf16 and k.attention_mma_supports(self.head_dim):
            # a step of single tokens: rotation, cache write, attention and the join in one kernel
            hpk = min(self.q_per_kv, 128)
            warps = (hpk + 15) // 16
            want = self._decode_splits(ctx, hpk)
            splits = max(s for s in k.DECODE_SPLITS if s <= want)
            tc = (slopes is None and self.window == 0 and getattr(ctx, "side_stream", None) is None
                  and k.attention_decode_tc_supports(self.head_dim, self.q_per_kv))
            # beside the feed-forward's weight stream (two graph branches) the attention only has to stay
            # off the critical path, and its blocks take SMs from the stream: 7/8 of the SMs at most
            if getattr(ctx, "side_stream", None) is not None:
                chunks = (self.q_per_kv + hpk - 1) // hpk
                sms = k.sm_count(self.build.device)
                want = min(want, max(1, (sms * 7 // 8) // (ctx.n_seqs * self.kv_heads * chunks)))
            teams = self._decode_teams(ctx, want, 4)
            if tc:
                # many query heads on a K/V head: they are the rows of one tcgen05 tile. Not while the
                # feed-forward streams its weights on the other graph branch: this kernel's 100 KB of
                # shared memory would keep those blocks off the SMs, where the mma.sync kernel's 58 KB
                # fit beside them
                o = k.attention_decode_tc(fused, k_pool, v_pool, batch, rope, self.kv_heads, self.q_per_kv,
                                          self.head_dim, self.scale, splits, write_cache=entry.writes_cache,
                                          n_teams=teams, interleaved=inter)
                return linear(k, o, self.p_out_weight, self.p_out_bias, add=add)
            o = k.attention_decode(fused, k_pool, v_pool, batch, rope, slopes, self.kv_heads, self.q_per_kv,
                                   self.head_dim, self.scale, self.window, hpk, warps, splits,
                                   write_cache=entry.writes_cache, key_split=self._decode_key_split(warps),
                                   n_teams=teams, interleaved=inter)
        else:
            q = k.split_rotate_store(fused, k_pool, v_pool, batch, None, self.kv_heads, self.q_per_kv,
                                     self.head_dim, write_cache=entry.writes_cache, rope=rope, interleaved=inter)
            o = self.attend(q, k_pool, v_pool, ctx, tiles, batch, slopes)
        return linear(k, o, self.p_out_weight, self.p_out_bias, add=add)

    def _decode_splits(self, ctx, hpk):
        """Blocks per (sequence, head chunk) for steps of single tokens: up to about two blocks on
        every SM, each with at least two pages of keys (measured: more, smaller blocks are slower
        at batch 64, and a second wave of blocks costs more than it brings)."""
        chunks = (self.q_per_kv + hpk - 1) // hpk
        blocks = ctx.n_seqs * self.kv_heads * chunks
        sms = self.build.kernels.sm_count(self.build.device)
        return max(1, min((2 * sms) // blocks, self._decode_pages(ctx) // 2, 64))

    def _decode_pages(self, ctx):
        pages = ctx.pages_hint
        if self.window > 0:
            pages = min(pages, self.window // self.build.kernels.PAGE + 2)
        return pages

    def _decode_teams(self, ctx, want, min_pages):
        """Clusters of blocks per (sequence, head chunk) in the decode kernels. A cluster holds 8 blocks;
        long sequences in a small batch need more to fill the SMs, each block with ``min_pages`` pages
        at least (16,384 keys, 71 heads on one K/V head, batch 1: 8 clusters of 8 blocks take 18 us
        against 57 us for one cluster)."""
        if want <= 8:
            return 1
        return max(1, min(want, self._decode_pages(ctx) // min_pages) // 8)

    def _decode_key_split(self, row_warps):
        """Groups of warps that share the keys of a page in the decode kernel. With few query heads
        per K/V head a block has one or two warps of rows, and each page is a chain of dependent
        work for them (4 query heads of size 128 per K/V head: 4 groups are 1.8 to 2 times faster);
        from three warps of rows on, more groups bring nothing."""
        if row_warps >= 3:
            return 1
        groups = 4 if self.head_dim > 64 else 2
        while groups > 1 and row_warps * groups > self.build.kernels.decode_max_warps(self.head_dim):
            groups //= 2
        return groups

    def attend(self, q, k_pool, v_pool, ctx, tiles, batch, slopes):
        k = self.build.kernels
        tokens = tiles.facts["mma_tokens"]
        if (q.dtype == self._bf16 and self.window == 0 and tokens == k.TC_TILE_TOKENS
                and k.attention_tc_supports(self.head_dim)):
            # long prompts: tcgen05 tensor cores, accumulators in tensor memory
            return k.attention_tc(q, k_pool, v_pool, batch, tiles.dev["mtile_seq"], tiles.dev["mtile_q0"],
                                  tiles.facts["n_mma_tiles"], self.kv_heads, self.scale, slopes)
        if q.dtype == self._bf16 and k.attention_mma_supports(self.head_dim):
            return self._attend_mma(q, k_pool, v_pool, ctx, tiles, batch, slopes)
        return k.attention_generic(q, k_pool, v_pool, batch, tiles.dev["tile_seq"], tiles.dev["tile_q0"],
                                   tiles.facts["n_tiles"], slopes, self.kv_heads, self.scale, self.window)

    def _attend_mma(self, q, k_pool, v_pool, ctx, tiles, batch, slopes):
        """Tile shape of the tensor-core kernel for this step. Single tokens: all heads of a K/V
        group in one tile, and the key pages divided among enough blocks to fill the device.
        Prompts: 128 rows of (tokens x heads of a group)."""
        k = self.build.kernels
        tokens = tiles.facts["mma_tokens"]
        if tokens == 1:
            hpk = min(self.q_per_kv, 128)
            warps = (hpk + 15) // 16
        else:
            warps = 8
            hpk = max(1, min(self.q_per_kv, 128 // tokens))
        splits = self._decode_splits(ctx, hpk) if tokens == 1 else 1
        return k.attention_mma(q, k_pool, v_pool, batch, tiles.dev["mtile_seq"], tiles.dev["mtile_q0"],
                               tiles.facts["n_mma_tiles"], slopes, self.kv_heads, self.scale, self.window, tokens, hpk,
                               warps, splits)
