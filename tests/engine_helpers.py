"""Helpers shared by the GPU tests: a cache with one attention entry, steps on raw kernels."""
import math

import torch

import plain_falcon as plain


def attention_case(K, dtype, heads, kv_heads, d, pasts, news, position="rotary", window=0, theta=10000.0,
                   seed=0, needle=None, mma=None, fused_decode=None, tc=False):
    """Run the split/rotate/store kernel and an attention function over random projections in two
    steps (first `pasts[b]` tokens, then `news[b]`) and return (engine output of the second step,
    plain output for the same rows) as float64 CPU tensors.

    needle=(b, key_pos): the last query of sequence b and the key at key_pos are made to align
    strongly, so that the row's output is essentially that key's value."""
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.attention import AttentionTiles
    from pytorch_transformers_b200.parts.base import CacheNeed
    from pytorch_transformers_b200.parts.position import alibi_slopes

    qpk = heads // kv_heads
    width = kv_heads * (qpk + 2) * d
    g = torch.Generator().manual_seed(seed)
    totals = [p + n for p, n in zip(pasts, news)]
    fused = [torch.randn(t, width, generator=g) for t in totals]
    if needle is not None:
        b, key_pos = needle
        f = fused[b].view(totals[b], kv_heads, qpk + 2, d)
        direction = torch.randn(d, generator=g)
        direction = direction / direction.norm()
        f[key_pos, :, qpk] = 0.0           # K of the needle: found only through the query's direction
        f[-1, :, :qpk] = 0.0
        if position == "rotary":
            # rotation would turn the two apart: use rotation-free models for needles
            raise ValueError("needle cases use position='alibi' or 'none'")
        f[key_pos, :, qpk] = 12.0 * direction
        f[-1, :, :qpk] = 12.0 * direction
    need = CacheNeed("window" if window else "full", kv_heads, d, window)
    max_tokens = sum((t + 63) // 64 * 64 for t in totals)
    cache = Cache([(0, need, None)], max_tokens, dtype, "cuda")
    slots = [cache.open() for _ in totals]
    inv_freq = None
    slopes = None
    if position == "rotary":
        inv_freq = (1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))).cuda()
    elif position == "alibi":
        slopes = alibi_slopes(heads).bfloat16().float().cuda()
    scale = 1.0 / math.sqrt(d)
    k_pool, v_pool, gi = cache.entry_storage(0)

    def step(ranges):
        live = [(s, r) for s, r in zip(slots, ranges) if r[1] > r[0]]
        idx = [i for i, r in enumerate(ranges) if r[1] > r[0]]
        toks = [[0] * (r[1] - r[0]) for _, r in live]
        ctx = StepContext(cache, [s for s, _ in live], toks, 1, [[] for _ in live], [AttentionTiles(K)])
        tiles = ctx.plan(AttentionTiles.plan_key)
        mma_tokens = tiles.facts["mma_tokens"]
        x = torch.cat([fused[i][r[0]:r[1]] for i, (_, r) in zip(idx, live)]).to(dtype).cuda().contiguous()
        if fused_decode is not None and mma_tokens == 1:
            # fused_decode = (heads per tile or None, splits[, key groups[, teams]]): the one-kernel decode path
            rope = K.rope_table(ctx.dev["tok_pos"], inv_freq) if inv_freq is not None else None
            hpk = fused_decode[0] or min(qpk, 128)
            if fused_decode[0] == "tc":
                # fused_decode = ("tc", splits[, teams]): the tcgen05 form of the one-kernel decode path
                out = K.attention_decode_tc(x, k_pool, v_pool, ctx.batch_c[gi], rope, kv_heads, qpk, d, scale,
                                            fused_decode[1], n_teams=fused_decode[2] if len(fused_decode) > 2 else 1)
                K.check_device_errors("cuda")
                ctx.commit()
                return out, idx
            out = K.attention_decode(x, k_pool, v_pool, ctx.batch_c[gi], rope, slopes, kv_heads, qpk, d, scale,
                                     window, hpk, (hpk + 15) // 16, fused_decode[1],
                                     key_split=fused_decode[2] if len(fused_decode) > 2 else 1,
                                     n_teams=fused_decode[3] if len(fused_decode) > 3 else 1)
            ctx.commit()
            return out, idx
        q = K.split_rotate_store(x, k_pool, v_pool, ctx.batch_c[gi], inv_freq, kv_heads, qpk, d)
        if tc:
            assert mma_tokens == K.TC_TILE_TOKENS
            out = K.attention_tc(q, k_pool, v_pool, ctx.batch_c[gi], tiles.dev["mtile_seq"], tiles.dev["mtile_q0"],
                                 tiles.facts["n_mma_tiles"], kv_heads, scale, slopes)
            K.check_device_errors("cuda")
        elif mma is None:
            out = K.attention_generic(q, k_pool, v_pool, ctx.batch_c[gi], tiles.dev["tile_seq"], tiles.dev["tile_q0"],
                                      tiles.facts["n_tiles"], slopes, kv_heads, scale, window)
        else:
            # mma = (heads per tile or None for "all that fit", splits)
            tokens = mma_tokens
            hpk = mma[0] or (min(qpk, 128) if tokens == 1 else max(1, min(qpk, 128 // tokens)))
            warps = (hpk * tokens + 15) // 16
            out = K.attention_mma(q, k_pool, v_pool, ctx.batch_c[gi], tiles.dev["mtile_seq"], tiles.dev["mtile_q0"],
                                  tiles.facts["n_mma_tiles"], slopes, kv_heads, scale, window, tokens, hpk, warps, mma[1])
        ctx.commit()
        return out, idx

    if any(p > 0 for p in pasts):
        step([(0, p) for p in pasts])
    out, idx = step([(p, t) for p, t in zip(pasts, totals)])
    cache.check()

    # plain: whole sequences, float64, on the values the engine saw (rounded to dtype)
    c = {"num_attention_heads": heads, "hidden_size": heads * d, "new_decoder_architecture": True,
         "num_kv_heads": kv_heads, "multi_query": False, "rope_theta": theta, "rope_scaling": None}
    refs = []
    for i in idx:
        f = fused[i].to(dtype).double()
        q, k, v = plain.split_heads(f, c)
        bias = None
        if position == "rotary":
            pos = torch.arange(totals[i])
            inv = plain.rope_inv_freq(c)
            q, k = plain.rotary(q, pos, inv), plain.rotary(k, pos, inv)
            if dtype == torch.bfloat16:      # the engine stores rotated K and passes rotated q in bfloat16
                q, k = q.to(dtype).double(), k.to(dtype).double()
        elif position == "alibi":
            bias = plain.alibi_bias(heads, totals[i], torch.float64)
        refs.append(plain_attention(q, k, v, bias, window)[pasts[i]:])
    return out.double().cpu(), torch.cat(refs)


def plain_attention(q, k, v, bias=None, window=0):
    """Causal (optionally windowed) attention of one whole sequence in the working dtype."""
    s, nh, d = q.shape
    qpk = nh // k.shape[1]
    i = torch.arange(s)
    visible = i[None, :] <= i[:, None]
    if window:
        visible &= i[None, :] > (i[:, None] - window)
    out = torch.empty(s, nh, d, dtype=q.dtype)
    for h in range(nh):
        sc = q[:, h] @ k[:, h // qpk].T
        if bias is not None:
            sc = sc + bias[h][None, :s]
        sc = (sc / math.sqrt(d)).masked_fill(~visible, float("-inf"))
        out[:, h] = torch.softmax(sc, -1) @ v[:, h // qpk]
    return out.reshape(s, nh * d)
