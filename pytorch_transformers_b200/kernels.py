"""Python face of the sm_100a kernel library: one function per entry point, torch tensors in.

Every function launches on the current CUDA stream of the tensors' device and raises
``KernelError`` if the entry point refuses its arguments. Nothing here computes on the host
and nothing falls back to torch: without a CUDA device, or without the compiled library, the
calls fail.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import native

PAGE = 64  # tokens of a cache page (PTB_PAGE in csrc/common.cuh)
# names (src/transformers/activations.py:200-228) -> the codes of csrc/common.cuh, the kernels' one table
ACTIVATIONS = {"none": 0, "gelu": 1, "gelu_new": 2, "gelu_pytorch_tanh": 2, "relu": 3}
NORM_KINDS = {"layernorm": 0, "rmsnorm": 1}
_ERRORS = {1: "unknown dtype code", 2: "a size that the kernel does not take", 3: "the CUDA launch failed",
           4: "a pointer or row size is not aligned as the kernel needs"}


class KernelError(RuntimeError):
    pass


class StepBatchC(ctypes.Structure):
    """Mirror of ``StepBatch`` in csrc/common.cuh."""
    _fields_ = [("tok_seq", ctypes.c_void_p), ("tok_pos", ctypes.c_void_p), ("seq_start", ctypes.c_void_p),
                ("seq_new", ctypes.c_void_p), ("seq_past", ctypes.c_void_p), ("pages", ctypes.c_void_p),
                ("pages_stride", ctypes.c_int), ("n_tokens", ctypes.c_int), ("n_seqs", ctypes.c_int)]


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


launches = 0  # entry points called so far (every one launches one kernel of this library)


def _check(code: int, what: str) -> None:
    global launches
    launches += 1
    if code != 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on a CUDA device only; got a tensor on " + str(t.device))
        if t is not None and not t.is_contiguous():
            raise KernelError("kernels take contiguous tensors")


_configured = False


def lib():
    global _configured
    L = native.library()
    if not _configured:
        for name in ("ptb_gather_rows", "ptb_norm", "ptb_bias_act", "ptb_residual", "ptb_to_float",
                     "ptb_linear_f32", "ptb_split_rotate_store", "ptb_attention_generic", "ptb_sample",
                     "ptb_attention_generic_tile_rows", "ptb_attention_mma", "ptb_attention_mma_supports",
                     "ptb_skinny_linear", "ptb_skinny_linear_max_rows", "ptb_skinny_linear_k_multiple",
                     "ptb_rope_table", "ptb_attention_decode", "ptb_attention_tc", "ptb_attention_tc_supports",
                     "ptb_attention_tc_tile_tokens", "ptb_tc_linear", "ptb_tc_linear_max_rows",
                     "ptb_tc_linear_k_multiple", "ptb_attention_decode_tc", "ptb_attention_decode_tc_supports",
                     "ptb_fill_normal", "ptb_selftest_bounded_wait", "ptb_scale", "ptb_selftest_mma_cadence"):
            getattr(L, name).restype = ctypes.c_int
        _configured = True
    return L


def generic_tile_rows() -> int:
    return 16  # BQ of csrc/attention_generic.cu (checked against the library in the GPU tests)


# ------------------------------------------------------------------------------------------------
def gather_rows(ids: torch.Tensor, table: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = table[ids[t]] (int32 ids). An id out of range sets bit 0 of ``status``."""
    _need_cuda(ids, table)
    out = torch.empty((ids.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    _check(lib().ptb_gather_rows(_dtype_code(table), _ptr(ids), _ptr(table), _ptr(out), ids.numel(),
                                 table.shape[1], table.shape[0], _ptr(status), _stream(table)), "gather_rows")
    return out


def norm(x: torch.Tensor, gain: torch.Tensor, bias: Optional[torch.Tensor], eps: float, kind: str = "layernorm",
         gain2: Optional[torch.Tensor] = None, bias2: Optional[torch.Tensor] = None,
         addend: Optional[torch.Tensor] = None):
    """LayerNorm / RMSNorm of rows; with ``gain2`` a second output from the same statistics. With
    ``addend`` the rows normalised are ``x + addend`` (one rounding), and that sum is returned first:
    ``(sum, y)`` or ``(sum, y, y2)``."""
    _need_cuda(x, gain, bias, gain2, bias2, addend)
    n, width = x.shape
    y1 = torch.empty_like(x)
    y2 = torch.empty_like(x) if gain2 is not None else None
    total = torch.empty_like(x) if addend is not None else None
    _check(lib().ptb_norm(_dtype_code(x), _ptr(x), _ptr(addend), _ptr(total), _ptr(gain), _ptr(bias), _ptr(y1),
                          _ptr(gain2), _ptr(bias2), _ptr(y2), n, width, ctypes.c_float(eps), NORM_KINDS[kind],
                          _stream(x)), "norm")
    outs = (y1,) if gain2 is None else (y1, y2)
    if addend is not None:
        return (total,) + outs
    return outs[0] if len(outs) == 1 else outs


def bias_act_(y: torch.Tensor, bias: Optional[torch.Tensor], act: str) -> torch.Tensor:
    """y = act(y + bias) in place."""
    _need_cuda(y, bias)
    _check(lib().ptb_bias_act(_dtype_code(y), _ptr(y), _ptr(bias), y.shape[0], y.shape[1], ACTIVATIONS[act],
                              _stream(y)), "bias_act")
    return y


def residual(x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x + (a + b), the sum formed in float32."""
    _need_cuda(x, a, b)
    out = torch.empty_like(x)
    _check(lib().ptb_residual(_dtype_code(x), _ptr(x), _ptr(a), _ptr(b), _ptr(out), ctypes.c_longlong(x.numel()),
                              _stream(x)), "residual")
    return out


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor in place (float32 product, one rounding)."""
    _need_cuda(x)
    _check(lib().ptb_scale(_dtype_code(x), _ptr(x), ctypes.c_float(factor), ctypes.c_longlong(x.numel()), _stream(x)),
           "scale")
    return x


def to_float(x: torch.Tensor) -> torch.Tensor:
    _need_cuda(x)
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    _check(lib().ptb_to_float(_dtype_code(x), _ptr(x), _ptr(out), ctypes.c_longlong(x.numel()), _stream(x)),
           "to_float")
    return out


def fill_normal(out: torch.Tensor, key: int, std: float, offset: float = 0.0, first: int = 0,
                round_bf16: bool = False) -> torch.Tensor:
    """out.flatten()[i] = offset + std * z(key, first + i): the device twin of weights/generator.py, bit for
    bit. ``round_bf16`` rounds a float32 tensor's values to what a bfloat16 tensor would hold."""
    _need_cuda(out)
    _check(lib().ptb_fill_normal(_dtype_code(out), _ptr(out), ctypes.c_ulonglong(out.numel()),
                                 ctypes.c_ulonglong(first), ctypes.c_ulonglong(key & (2 ** 64 - 1)),
                                 ctypes.c_double(std), ctypes.c_double(offset), 1 if round_bf16 else 0,
                                 _stream(out)), "fill_normal")
    return out


def linear_f32(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none"):
    """act(x @ w.T + bias) in true float32 on the CUDA cores."""
    _need_cuda(x, w, bias)
    if x.dtype != torch.float32 or w.dtype != torch.float32:
        raise KernelError("linear_f32 takes float32 tensors")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"linear_f32: x is [{m}, {k}] but w is {list(w.shape)}")
    y = torch.empty((m, n), dtype=torch.float32, device=x.device)
    _check(lib().ptb_linear_f32(_ptr(x), _ptr(w), _ptr(bias), _ptr(y), m, n, k, ACTIVATIONS[act], _stream(x)),
           "linear_f32")
    return y


def rope_table(tok_pos: torch.Tensor, inv_freq: torch.Tensor):
    """(cos, sin) of position * inv_freq for every token of a step: float32 [tokens, pairs] each."""
    _need_cuda(tok_pos, inv_freq)
    n, pairs = tok_pos.numel(), inv_freq.numel()
    table = torch.empty((2, n, pairs), dtype=torch.float32, device=inv_freq.device)
    _check(lib().ptb_rope_table(_ptr(tok_pos), _ptr(inv_freq), _ptr(table[0]), _ptr(table[1]), n, pairs,
                                _stream(inv_freq)), "rope_table")
    return table[0], table[1]


def split_rotate_store(fused: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                       batch: StepBatchC, inv_freq: Optional[torch.Tensor], kv_heads: int, q_per_kv: int,
                       head_dim: int, write_cache: bool = True, rope=None, interleaved: bool = False) -> torch.Tensor:
    """Fused projection -> rotated queries [tokens, heads, head_dim]; K (rotated) and V go to the pools.
    The rotation comes from ``inv_freq`` (angles computed in the kernel) or from ``rope`` = (cos, sin)
    tables of ``rope_table`` for this step's tokens; the pairs are (i, i + pairs) of a head's first
    2 * pairs dims, or (2 i, 2 i + 1) with ``interleaved``."""
    _need_cuda(fused, k_pool, v_pool, inv_freq)
    n = fused.shape[0]
    q = torch.empty((n, kv_heads * q_per_kv, head_dim), dtype=fused.dtype, device=fused.device)
    if fused.shape[1] != kv_heads * (q_per_kv + 2) * head_dim:
        raise KernelError(f"fused projection has width {fused.shape[1]}, expected "
                          f"{kv_heads * (q_per_kv + 2) * head_dim}")
    pairs = 0 if inv_freq is None else inv_freq.numel()
    cos = sin = None
    if rope is not None:
        cos, sin = rope
        pairs = cos.shape[1]
        inv_freq = None
    _check(lib().ptb_split_rotate_store(_dtype_code(fused), _ptr(fused), _ptr(q), _ptr(k_pool), _ptr(v_pool),
                                        ctypes.byref(batch), _ptr(inv_freq), _ptr(cos), _ptr(sin), pairs, kv_heads,
                                        q_per_kv, head_dim, 1 if write_cache else 0, 1 if interleaved else 0,
                                        _stream(fused)),
           "split_rotate_store")
    return q


def attention_generic(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatchC,
                      tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int,
                      slopes: Optional[torch.Tensor], kv_heads: int, scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of the step's tokens over the paged cache; returns [tokens, heads * head_dim]."""
    _need_cuda(q, k_pool, v_pool, tile_seq, tile_q0, slopes)
    n, heads, head_dim = q.shape
    out = torch.empty((n, heads * head_dim), dtype=q.dtype, device=q.device)
    _check(lib().ptb_attention_generic(_dtype_code(q), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out),
                                       ctypes.byref(batch), _ptr(tile_seq), _ptr(tile_q0), n_tiles, _ptr(slopes),
                                       heads, kv_heads, head_dim, ctypes.c_float(scale), window, _stream(q)),
           "attention_generic")
    return out


DECODE_SPLITS = (1, 2, 3, 4, 5, 6, 7, 8)   # ptb_attention_decode: the blocks of a split set form one cluster
DECODE_KEY_SPLITS = (1, 2, 4)              # groups of warps that share a page's keys


def decode_max_warps(head_dim: int) -> int:
    """Warps of a block of attention_decode: row warps times key groups."""
    return 10 if head_dim == 64 else 8


def attention_decode(fused: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatchC, rope,
                     slopes: Optional[torch.Tensor], kv_heads: int, q_per_kv: int, head_dim: int, scale: float,
                     window: int, heads_per_tile: int, warps: int, n_splits: int, write_cache: bool = True,
                     key_split: int = 1, n_teams: int = 1, interleaved: bool = False):
    """One kernel for the attention of a step of single tokens: rotate q and k of each new token, put
    k and v into the cache, attend over the cache (all heads of a K/V group in one tile of ``warps``
    x 16 rows, key pages divided among ``n_splits`` blocks of one cluster, the keys of a page among
    ``key_split`` groups of warps, all joined through (distributed) shared memory; ``n_teams`` such
    clusters share the pages of a long sequence and join through a workspace in global memory).
    Returns [tokens, heads * head_dim]."""
    _need_cuda(fused, k_pool, v_pool, slopes)
    if fused.dtype != torch.bfloat16:
        raise KernelError("attention_decode takes bfloat16 tensors")
    n = fused.shape[0]
    heads = kv_heads * q_per_kv
    if fused.shape[1] != kv_heads * (q_per_kv + 2) * head_dim:
        raise KernelError(f"fused projection has width {fused.shape[1]}, expected "
                          f"{kv_heads * (q_per_kv + 2) * head_dim}")
    out = torch.empty((n, heads * head_dim), dtype=fused.dtype, device=fused.device)
    cos, sin = rope if rope is not None else (None, None)
    pairs = 0 if cos is None else cos.shape[1]
    parts = tickets = None
    part_floats = n_tickets = 0
    if n_teams > 1:
        groups = n * kv_heads * ((q_per_kv + heads_per_tile - 1) // heads_per_tile)
        if groups * n_splits > DECODE_TICKETS:
            raise KernelError("attention_decode: too many (sequence, head chunk, split) triples for the ticket buffer")
        part_floats = groups * n_teams * heads_per_tile * (head_dim + 2)
        parts = torch.empty(part_floats, dtype=torch.float32, device=fused.device)
        n_tickets = groups * n_splits
        tickets = _tickets(n_tickets, fused.device)
    _check(lib().ptb_attention_decode(_ptr(fused), _ptr(k_pool), _ptr(v_pool), _ptr(out), ctypes.byref(batch),
                                      _ptr(cos), _ptr(sin), pairs, 1 if interleaved else 0, _ptr(slopes), heads, kv_heads,
                                      head_dim,
                                      heads_per_tile, n_splits, n_teams, warps, key_split, ctypes.c_float(scale),
                                      window, 1 if write_cache else 0, _ptr(parts), ctypes.c_size_t(part_floats),
                                      _ptr(tickets), n_tickets, _stream(fused)),
           "attention_decode")
    return out


def attention_decode_tc_supports(head_dim: int, q_per_kv: int) -> bool:
    return bool(lib().ptb_attention_decode_tc_supports(int(head_dim), int(q_per_kv)))


def attention_decode_tc(fused: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatchC, rope,
                        kv_heads: int, q_per_kv: int, head_dim: int, scale: float, n_splits: int,
                        write_cache: bool = True, n_teams: int = 1, interleaved: bool = False):
    """The attention of a step of single tokens on the tcgen05 tensor cores, for K/V heads that serve
    33 to 128 query heads of size 64: the query heads of a group are the rows of one tile, S, P and O
    live in tensor memory, pages come by TMA, ``n_splits`` blocks of one cluster share a sequence's
    pages and join through distributed shared memory; ``n_teams`` such clusters share the pages of a
    long sequence and join through a workspace in global memory. No score bias, no window.
    Returns [tokens, heads * head_dim]."""
    _need_cuda(fused, k_pool, v_pool)
    if fused.dtype != torch.bfloat16:
        raise KernelError("attention_decode_tc takes bfloat16 tensors")
    n = fused.shape[0]
    heads = kv_heads * q_per_kv
    if fused.shape[1] != kv_heads * (q_per_kv + 2) * head_dim:
        raise KernelError(f"fused projection has width {fused.shape[1]}, expected "
                          f"{kv_heads * (q_per_kv + 2) * head_dim}")
    if not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.shape != v_pool.shape:
        raise KernelError("attention_decode_tc takes the contiguous K and V pools of one cache entry")
    out = torch.empty((n, heads * head_dim), dtype=fused.dtype, device=fused.device)
    cos, sin = rope if rope is not None else (None, None)
    pairs = 0 if cos is None else cos.shape[1]
    parts = tickets = None
    part_floats = n_tickets = 0
    if n_teams > 1:
        if n * kv_heads * n_splits > DECODE_TICKETS:
            raise KernelError("attention_decode_tc: too many (sequence, K/V head, split) triples for the ticket buffer")
        part_floats = n * kv_heads * n_teams * q_per_kv * (head_dim + 2)
        parts = torch.empty(part_floats, dtype=torch.float32, device=fused.device)
        n_tickets = n * kv_heads * n_splits
        tickets = _tickets(n_tickets, fused.device)
    _check(lib().ptb_attention_decode_tc(_ptr(fused), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(out),
                                         ctypes.byref(batch), _ptr(cos), _ptr(sin), pairs, 1 if interleaved else 0, heads,
                                         kv_heads, head_dim,
                                         n_splits, n_teams, ctypes.c_float(scale), 1 if write_cache else 0,
                                         _ptr(parts), ctypes.c_size_t(part_floats), _ptr(tickets), n_tickets,
                                         _ptr(error_flag(fused.device)), _stream(fused)), "attention_decode_tc")
    return out


DECODE_TICKETS = 8192      # most (sequence, K/V head, split) triples of one decode attention launch
TICKET_ARENA = 1 << 18     # int32 words per device
_ticket_arenas = {}


def _tickets(n: int, device) -> torch.Tensor:
    """``n`` int32 zeros for a launch whose blocks count their arrivals; the kernel leaves them zero.
    Two launches that run at the same time (the two branches of a block, side by side in one graph)
    must not count in the same words, so every launch takes the next stretch of a zeroed arena, which
    wraps around after tens of launches; launches that far apart in a stream or a graph depend on
    one another and never overlap. The arena is allocated at a device's first launch, which is never
    inside a stream capture (a captured step has run once plainly before)."""
    device = torch.device(device)
    arena = _ticket_arenas.get(device)
    if arena is None:
        arena = _ticket_arenas[device] = [torch.zeros(TICKET_ARENA, dtype=torch.int32, device=device), 0]
    n = (n + 31) // 32 * 32
    if n > TICKET_ARENA:
        raise KernelError(f"a launch asks for {n} tickets, more than the arena's {TICKET_ARENA}")
    if arena[1] + n > TICKET_ARENA:
        arena[1] = 0
    out = arena[0][arena[1]:arena[1] + n]
    arena[1] += n
    return out


_error_flags = {}
TC_TILE_TOKENS = 128  # ptb_attention_tc_tile_tokens()


def error_flag(device) -> torch.Tensor:
    """Device int32 word that kernels with bounded waits raise when a wait runs out."""
    device = torch.device(device)
    if device not in _error_flags:
        _error_flags[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[device]


def check_device_errors(device) -> None:
    """Raise if a kernel has reported that one of its bounded waits ran out (synchronises)."""
    device = torch.device(device)
    flag = _error_flags.get(device)
    if flag is not None:
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            raise KernelError(f"a kernel gave up waiting inside its pipeline (code {code}): its results are void")


def selftest_mma_cadence(device, n: int, reps: int = 1000, a_in_tmem: bool = False, blocks: int = 1) -> float:
    """Clocks per tcgen05.mma (M = 128, K = 16, N = ``n``) when one thread of each of ``blocks`` blocks issues
    ``4 * reps`` of them back to back on operands that sit in shared (or tensor) memory."""
    device = torch.device(device)
    clocks = torch.zeros(1, dtype=torch.int64, device=device)
    _check(lib().ptb_selftest_mma_cadence(int(n), int(reps), 1 if a_in_tmem else 0, int(blocks), _ptr(clocks),
                                          _ptr(error_flag(device)),
                                          ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)),
           "selftest_mma_cadence")
    return float(clocks.item()) / (4 * reps)


def selftest_bounded_wait(device, tries: int = 1000) -> torch.Tensor:
    """Launch a kernel that waits, at most ``tries`` times, on a barrier at which nobody arrives: the wait
    runs out and raises the device's error flag, as a tcgen05 kernel does whose copy never lands.
    Returns an int32 word that the kernel sets to 1 when it gave up. ``check_device_errors`` then raises."""
    device = torch.device(device)
    gave_up = torch.zeros(1, dtype=torch.int32, device=device)
    _check(lib().ptb_selftest_bounded_wait(int(tries), _ptr(error_flag(device)), _ptr(gave_up),
                                           ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)),
           "selftest_bounded_wait")
    return gave_up


def attention_tc_supports(head_dim: int) -> bool:
    return bool(lib().ptb_attention_tc_supports(int(head_dim)))


def attention_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatchC,
                 tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, kv_heads: int, scale: float,
                 slopes: Optional[torch.Tensor] = None):
    """Causal prompt attention on tcgen05 tensor cores with accumulators in tensor memory: bfloat16,
    head size 64 or 128, tiles of 128 tokens, no window; ``slopes`` [heads] float32: per-head score
    slopes (ALiBi). Returns [tokens, heads * head_dim]."""
    _need_cuda(q, k_pool, v_pool, tile_seq, tile_q0, slopes)
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_tc takes bfloat16 tensors")
    n, heads, head_dim = q.shape
    out = torch.empty((n, heads * head_dim), dtype=q.dtype, device=q.device)
    if not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.shape != v_pool.shape:
        raise KernelError("attention_tc takes the contiguous K and V pools of one cache entry")
    _check(lib().ptb_attention_tc(_ptr(q), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(out), ctypes.byref(batch), _ptr(tile_seq),
                                  _ptr(tile_q0), n_tiles, _ptr(slopes), heads, kv_heads, head_dim, ctypes.c_float(scale),
                                  _ptr(error_flag(q.device)), _stream(q)), "attention_tc")
    return out


def attention_tc_pairs(mode) -> None:
    """For measurements and tests. ``attention_tc`` with head size 128 puts two heads of a K/V group in one
    block where the pairs fill the device (mode 1 or True, the default); 0 or False: never; 2: wherever a
    group has two heads or more."""
    lib().ptb_attention_tc_pairs(int(mode))


def attention_mma_supports(head_dim: int) -> bool:
    return bool(lib().ptb_attention_mma_supports(int(head_dim)))


def attention_mma(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatchC,
                  tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, slopes: Optional[torch.Tensor],
                  kv_heads: int, scale: float, window: int, tokens_per_tile: int, heads_per_tile: int, warps: int,
                  n_splits: int, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tensor-core attention over the paged cache (bfloat16). A tile holds ``tokens_per_tile`` tokens
    x ``heads_per_tile`` heads of one K/V group in ``warps`` x 16 rows; with ``n_splits`` > 1 the key
    pages are divided among blocks and joined by a second kernel (``scratch``: float32 workspace)."""
    _need_cuda(q, k_pool, v_pool, tile_seq, tile_q0, slopes, scratch)
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_mma takes bfloat16 tensors")
    n, heads, head_dim = q.shape
    out = torch.empty((n, heads * head_dim), dtype=q.dtype, device=q.device)
    if n_splits > 1:
        need = attention_mma_scratch_floats(n_tiles, heads, kv_heads, heads_per_tile, n_splits, warps, head_dim)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        elif scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"attention_mma: scratch of {need} float32 values needed")
    _check(lib().ptb_attention_mma(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(scratch),
                                   ctypes.byref(batch), _ptr(tile_seq), _ptr(tile_q0), n_tiles, _ptr(slopes),
                                   heads, kv_heads, head_dim, heads_per_tile, tokens_per_tile, n_splits, warps,
                                   ctypes.c_float(scale), window, _stream(q)), "attention_mma")
    if n_splits > 1:
        global launches
        launches += 1   # the kernel that joins the splits
    return out


def attention_mma_scratch_floats(n_tiles: int, heads: int, kv_heads: int, heads_per_tile: int, n_splits: int,
                                 warps: int, head_dim: int) -> int:
    if n_splits <= 1:
        return 0
    chunks = (heads // kv_heads + heads_per_tile - 1) // heads_per_tile
    return n_tiles * kv_heads * chunks * n_splits * warps * 16 * (head_dim + 2)


def sample(logits: torch.Tensor, work: torch.Tensor, out: torch.Tensor, *, do_sample: bool, temperature: float = 1.0,
           top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
           history: Optional[torch.Tensor] = None, history_len: Optional[torch.Tensor] = None,
           suppress: Optional[torch.Tensor] = None, seed: int = 0, streams: Optional[torch.Tensor] = None,
           counters: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Select one token per row of float32 logits into ``out`` (int32). ``work`` is scratch of the
    logits' shape; ``streams`` and ``counters`` (int64 per row) key the uniform draw."""
    _need_cuda(logits, work, out, history, history_len, suppress, streams, counters)
    if logits.dtype != torch.float32 or work.dtype != torch.float32 or out.dtype != torch.int32:
        raise KernelError("sample takes float32 logits and scratch and an int32 output")
    rows, vocab = logits.shape
    if work.numel() < logits.numel() or out.numel() < rows:
        raise KernelError("sample: scratch or output too small")
    if do_sample and (streams is None or counters is None):
        raise KernelError("sample: sampling needs the per-row stream and counter tensors")
    _check(lib().ptb_sample(_ptr(logits), _ptr(work), _ptr(out), rows, vocab, 1 if do_sample else 0,
                            ctypes.c_float(temperature), int(top_k), ctypes.c_float(top_p), ctypes.c_float(min_p),
                            ctypes.c_float(repetition_penalty), _ptr(history), _ptr(history_len),
                            0 if history is None else history.shape[1], _ptr(suppress),
                            0 if suppress is None else suppress.numel(), ctypes.c_ulonglong(seed & (2 ** 64 - 1)),
                            _ptr(streams), _ptr(counters), _stream(logits)), "sample")
    return out


SKINNY_MAX_ROWS = 32   # ptb_skinny_linear_max_rows()
SKINNY_K_MULTIPLE = 32  # ptb_skinny_linear_k_multiple()


# Rows beyond which the library product is faster inside a step (12 rows: 3.40 against 3.49 ms a step;
# 16 rows: 3.51 against 3.22).
SKINNY_BEST_ROWS = 12
# A matrix of tens of thousands of rows (the vocabulary's) runs alone in the step, and there the library
# reads it faster from 5 rows on (591 MB, float32 out, 8 rows: 92.7 against 86.9 us).
SKINNY_TALL_ROWS = 32768
SKINNY_BEST_ROWS_TALL = 4


def skinny_linear_takes(rows: int, k: int) -> bool:
    return 0 < rows <= SKINNY_MAX_ROWS and k % SKINNY_K_MULTIPLE == 0


def skinny_linear_preferred(rows: int, k: int, n: int = 0) -> bool:
    best = SKINNY_BEST_ROWS_TALL if n >= SKINNY_TALL_ROWS else SKINNY_BEST_ROWS
    return 0 < rows <= best and k % SKINNY_K_MULTIPLE == 0


def skinny_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
                  add: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """act(x @ w.T + bias) + add for up to 32 rows of bfloat16 x: one pass over w at memory speed,
    float32 accumulation and epilogue; the result is bfloat16 or float32."""
    _need_cuda(x, w, bias, add)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (add is not None and add.dtype != torch.bfloat16):
        raise KernelError("skinny_linear takes bfloat16 x, w and add")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or (add is not None and tuple(add.shape) != (m, n)):
        raise KernelError(f"skinny_linear: shapes x {list(x.shape)}, w {list(w.shape)} do not fit")
    y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    ybf, yf = (y, None) if out_dtype == torch.bfloat16 else (None, y)
    # where the tiles of w do not divide evenly over the SMs the kernel divides K among several blocks per
    # tile; their partial sums meet in scratch memory, a zeroed ticket per tile says who is last
    need = _skinny_scratch_floats(m, n, k)
    scratch = torch.empty(need, dtype=torch.float32, device=x.device) if need else None
    n_tickets = (n + 15) // 16 if need else 0        # a ticket per tile of weight rows; tiles have 16 rows or more
    tickets = _tickets(n_tickets, x.device) if need else None
    _check(lib().ptb_skinny_linear(_ptr(x), _ptr(w), _ptr(bias), _ptr(add), _ptr(ybf), _ptr(yf), m, n, k,
                                   ACTIVATIONS[act], _ptr(scratch), ctypes.c_size_t(need), _ptr(tickets),
                                   n_tickets, _stream(x)), "skinny_linear")
    return y


_skinny_scratch_cache = {}


def _skinny_scratch_floats(m: int, n: int, k: int) -> int:
    key = (m, n, k)
    if key not in _skinny_scratch_cache:
        fn = lib().ptb_skinny_linear_scratch
        fn.restype = ctypes.c_longlong
        _skinny_scratch_cache[key] = int(fn(m, n, k))
    return _skinny_scratch_cache[key]


_sm_count = {}


def sm_count(device) -> int:
    """Multiprocessors of ``device`` (148 on a B200); without a CUDA device, the B200's count."""
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        return 148
    if device not in _sm_count:
        _sm_count[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[device]


# A step of few tokens is bound by the read of the weights, and a mixer's small kernels can hide under
# the feed-forward's weight stream on a second stream. Two limits say how long that pays:
# rows of the step (beyond them the linear layers are no longer pure weight streams; two branches
# against one at 48 rows: 4.19 against 4.49 ms a step, at 64 rows: 4.44 against 4.25), and the bytes of
# keys and values that one attention layer reads in the step: once they are tens of megabytes the
# attention competes with the weight stream instead of hiding under it (34 MB: 3.43 against 3.85 ms;
# 42 MB: 4.49 against 4.24). Heads wider than 64 need the decode kernel's large page ring, which keeps
# the stream's blocks off the SMs earlier (17 MB: 5.39 against 5.55 ms; 34 MB: 7.80 against 5.80).
WEIGHT_STREAM_MAX_ROWS = 48
DECODE_BESIDE_MAX_KV_BYTES = 40 << 20
DECODE_BESIDE_MAX_KV_BYTES_WIDE_HEADS = 24 << 20


def decode_attention_fits_beside(kv_bytes: int, head_dim: int) -> bool:
    """May a decode attention that reads ``kv_bytes`` of keys and values run beside a weight stream?"""
    return kv_bytes <= (DECODE_BESIDE_MAX_KV_BYTES if head_dim <= 64 else DECODE_BESIDE_MAX_KV_BYTES_WIDE_HEADS)


TC_LINEAR_MAX_ROWS = 128   # ptb_tc_linear_max_rows()
TC_LINEAR_K_MULTIPLE = 8   # ptb_tc_linear_k_multiple()


def tc_linear_takes(rows: int, k: int) -> bool:
    return 0 < rows <= TC_LINEAR_MAX_ROWS and k % TC_LINEAR_K_MULTIPLE == 0


def tc_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
              add: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """act(x @ w.T + bias) + add for up to 128 rows of bfloat16 x on the tcgen05 tensor cores: the
    weights stream once through shared memory (TMA), the sums stay in tensor memory, and bias,
    activation and the sum with ``add`` happen in the float32 epilogue. Result bfloat16 or float32."""
    _need_cuda(x, w, bias, add)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (add is not None and add.dtype != torch.bfloat16):
        raise KernelError("tc_linear takes bfloat16 x, w and add")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or (add is not None and tuple(add.shape) != (m, n)):
        raise KernelError(f"tc_linear: shapes x {list(x.shape)}, w {list(w.shape)} do not fit")
    if not x.is_contiguous() or not w.is_contiguous() or (add is not None and not add.is_contiguous()):
        raise KernelError("tc_linear takes contiguous tensors")
    dev = x.device
    y = torch.empty((m, n), dtype=out_dtype, device=dev)
    ybf, yf = (y, None) if out_dtype == torch.bfloat16 else (None, y)
    _check(lib().ptb_tc_linear(_ptr(x), _ptr(w), _ptr(bias), _ptr(add), _ptr(ybf), _ptr(yf), m, n, k,
                               ACTIVATIONS[act], sm_count(dev), _ptr(error_flag(dev)), _stream(x)), "tc_linear")
    return y


def matmul_nt(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
              add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Library matrix product x @ w.T (+ add) for the bfloat16 path (cuBLAS through torch), where the
    reference's engine uses the same library. float32 inputs are refused: the float32 path has
    its own kernel (linear_f32)."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("matmul_nt is the bfloat16 library product; float32 goes through linear_f32")
    _need_cuda(x, w)
    if add is not None:
        # the library's own epilogue adds in float32 and rounds once (beta = 1)
        if out_dtype not in (None, torch.bfloat16) or add.dtype != torch.bfloat16 or tuple(add.shape) != (x.shape[0], w.shape[0]):
            raise KernelError("matmul_nt adds a bfloat16 tensor of the result's shape to a bfloat16 result")
        return torch.addmm(add, x, w.t())
    if out_dtype is None or out_dtype == torch.bfloat16:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)
