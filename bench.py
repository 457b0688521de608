"""Benchmark of the headline metric: decoded tokens per second of a Falcon-7B-shaped model in
bfloat16 with random weights on one B200, batch 8 at context 2,048; plus prefill of 2,048
tokens, decode at batch 1 and 64, the HBM roofline of the decode step, and the same decode rate
end to end through ``generate`` (host tokens in and out).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

One JSON line on stdout. A "step" is one decode step of the whole batch. Timing: CUDA events on
the launching stream around exactly K steps after W warm-up steps, a synchronize on both sides;
every step reads all weights (13.8 GB, far beyond the 126 MB L2), so no cache flush is needed
between steps. SM clocks and throttle reasons are sampled with nvidia-smi during the timed
region. ``--impl reference`` runs the reference's own FalconForCausalLM.generate from
baseline/_ref on the same shapes.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALCON_7B = dict(vocab_size=65024, hidden_size=4544, num_hidden_layers=32, num_attention_heads=71,
                 multi_query=True, parallel_attn=True, new_decoder_architecture=False, bias=False, alibi=False,
                 rope_theta=10000.0, layer_norm_epsilon=1e-5, max_position_embeddings=2048,
                 tie_word_embeddings=True, activation="gelu")
# the other two shapes that the reference's Falcon family has (for `--only decode --shape ...`)
FALCON_11B = dict(vocab_size=65024, hidden_size=4096, num_hidden_layers=60, num_attention_heads=32, num_kv_heads=8,
                  new_decoder_architecture=True, num_ln_in_parallel_attn=1, ffn_hidden_size=16384,
                  rope_theta=500042.0, bias=False, alibi=False, layer_norm_epsilon=1e-5,
                  max_position_embeddings=8192, tie_word_embeddings=True, activation="gelu")
FALCON_40B = dict(vocab_size=65024, hidden_size=8192, num_hidden_layers=60, num_attention_heads=128, num_kv_heads=8,
                  new_decoder_architecture=True, ffn_hidden_size=32768, rope_theta=10000.0, bias=False, alibi=False,
                  layer_norm_epsilon=1e-5, max_position_embeddings=2048, tie_word_embeddings=False,
                  activation="gelu")
SHAPES = {"7b": FALCON_7B, "11b": FALCON_11B, "40b": FALCON_40B}
CONTEXT = 2048
PREFILL_TOKENS = 2048
SETTLE_STEPS = 40     # untimed decode steps after a prefill, before the warm-up steps (see run_ours)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained") or raw["bf16_tflops"]),
                    "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(int(s[0]))
                mx.append(int(s[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not mhz:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": int(statistics.median(mhz)), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


def workload_config(layers, batch):
    """What is run, in the same words for both arms: the layer sizes of Falcon-7B, the batch, the context."""
    h, nh, kvh, d, f, v = shape_sizes(FALCON_7B)
    return {"model": "falcon-7b-shape", "layers": layers, "layers_of_config": FALCON_7B["num_hidden_layers"],
            "hidden": h, "heads": nh, "kv_heads": kvh, "head_dim": d, "ffn": f, "vocab": v, "global_batch": batch,
            "seq_len": CONTEXT, "prompt_tokens": CONTEXT, "weights": "random seed 0", "tokens": "uniform seed 0",
            "parallelism": "none", "sampling": "greedy",
            "l2": "inputs larger than L2 (all weights read per step)"}


def shape_sizes(c):
    """(hidden, heads, K/V heads, head size, feed-forward width, vocabulary) of a shape dictionary."""
    h, nh, v = c["hidden_size"], c["num_attention_heads"], c["vocab_size"]
    f = c.get("ffn_hidden_size") or 4 * h
    kvh = c.get("num_kv_heads", 1) if c.get("new_decoder_architecture") else (1 if c.get("multi_query", True) else nh)
    return h, nh, kvh, h // nh, f, v


def falcon_param_count(c, layers):
    """Weights that a step reads: the layers' matrices and norm vectors and the head matrix (tied or not,
    it is read once; of the embedding table a step reads a row per token). Also the count of one layer."""
    h, nh, kvh, d, f, v = shape_sizes(c)
    norms = 2 if (c.get("new_decoder_architecture") and c.get("num_ln_in_parallel_attn", 2) != 1) or \
        not (c.get("new_decoder_architecture") or c.get("parallel_attn", True)) else 1
    per_layer = (nh + 2 * kvh) * d * h + h * h + 2 * f * h + norms * 2 * h
    return layers * per_layer + v * h + 2 * h, per_layer


def decode_bytes(c, layers, batch, context):
    """Bytes a decode step has to read: every weight it uses once and the cached keys and values of the
    live requests, in bfloat16."""
    h, nh, kvh, d, f, v = shape_sizes(c)
    params, _ = falcon_param_count(c, layers)
    kv = batch * context * layers * 2 * kvh * d * 2
    return 2 * params + kv


def prefill_flops(c, layers, tokens):
    h, nh, kvh, d, f, v = shape_sizes(c)
    gemm = 2 * tokens * layers * ((nh + 2 * kvh) * d * h + h * h + 2 * f * h)
    attn = layers * nh * 2 * 2 * d * tokens * (tokens + 1) / 2      # QK^T and PV over the causal half
    head = 2 * v * h
    return gemm + attn + head


class NoCollection:
    """The engine's guard for stream captures (no cyclic garbage collection inside), looked up when used so
    that `bench.py --gpus 2` and `--impl reference` need not import the package."""

    def __enter__(self):
        from pytorch_transformers_b200.engine.model import NoCollection as Guard
        self.guard = Guard()
        return self.guard.__enter__()

    def __exit__(self, *exc):
        return self.guard.__exit__(*exc)


def run_sample(args):
    """Device time of the selection kernel for the ways of sampling, `--batch` rows of the 7B vocabulary,
    20 launches captured in a CUDA graph (no host time); rows of scale 3 are flat, of scale 6 peaked."""
    import torch

    from pytorch_transformers_b200 import kernels

    torch.cuda.set_device(0)
    rows, vocab = args.batch, SHAPES["7b"]["vocab_size"]
    gen = torch.Generator(device="cuda").manual_seed(0)
    base = torch.randn(rows, vocab, device="cuda", generator=gen)
    work = torch.empty_like(base)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    streams = torch.arange(rows, dtype=torch.int64, device="cuda")
    counters = torch.zeros(rows, dtype=torch.int64, device="cuda")
    cases = {"greedy": (3.0, dict(do_sample=False)), "temperature": (3.0, dict(do_sample=True, temperature=0.8)),
             "top_k 50": (3.0, dict(do_sample=True, top_k=50)),
             "top_k 50 top_p 0.9": (3.0, dict(do_sample=True, top_k=50, top_p=0.9, temperature=0.7)),
             "top_k 2000": (3.0, dict(do_sample=True, top_k=2000)),
             "top_p 0.9 peaked": (6.0, dict(do_sample=True, top_p=0.9)),
             "top_p 0.9 flat": (3.0, dict(do_sample=True, top_p=0.9)), "min_p 0.05": (3.0, dict(do_sample=True, min_p=0.05))}
    result = {"only": "sample", "rows": rows, "vocab": vocab, "unit": "us per launch"}
    side = torch.cuda.Stream()
    for name, (scale, opt) in cases.items():
        logits = base * scale
        launch = lambda: kernels.sample(logits, work, out, seed=1, streams=streams, counters=counters, **opt)
        with torch.cuda.stream(side):
            for _ in range(3):
                launch()
            graph = torch.cuda.CUDAGraph()
            with NoCollection(), torch.cuda.graph(graph, stream=side):
                for _ in range(20):
                    launch()
            graph.replay()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(5):
                graph.replay()
            t1.record()
        torch.cuda.synchronize()
        result[name] = round(t0.elapsed_time(t1) * 10.0, 1)   # ms for 100 launches -> us for one
    print(json.dumps(result))
    return 0


def run_decode_attention(args):
    """Device time of the two decode attention kernels alone (20 launches in a CUDA graph), `--batch`
    sequences of `--context` cached keys with the heads of `--shape`, for blocks a cluster x clusters a
    sequence."""
    import math

    import torch

    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200 import kernels as K
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.base import CacheNeed

    torch.cuda.set_device(0)
    cfg = ptb.FalconConfig.from_dict(SHAPES[args.shape])
    kv, d, qpk, rows, keys = cfg.kv_heads_eff, cfg.head_dim, cfg.q_per_kv, args.batch, args.context
    cache = Cache([(0, CacheNeed("full", kv, d, 0), None)], rows * (keys + 64), torch.bfloat16, "cuda")
    slots = [cache.open() for _ in range(rows)]
    for slot in slots:
        cache.reserve(slot, keys)
        cache.commit(slot, keys)
    k_pool, v_pool, group = cache.entry_storage(0)
    k_pool.normal_()
    v_pool.normal_()
    ctx = StepContext(cache, slots, [[0]] * rows, 1, [[]] * rows)
    fused = torch.randn(rows, kv * (qpk + 2) * d, device="cuda", dtype=torch.bfloat16)
    rope = K.rope_table(ctx.dev["tok_pos"], (1.0 / (10000 ** (torch.arange(0, d, 2).float() / d))).cuda())
    hpk = min(qpk, 128)
    warps, scale, batch = (hpk + 15) // 16, 1 / math.sqrt(d), ctx.batch_c[group]
    key_split = 1 if warps >= 3 else min(4 if d > 64 else 2, K.decode_max_warps(d) // warps)
    result = {"only": "decode-attention", "shape": args.shape, "batch": rows, "context": keys, "unit": "us per launch"}
    side = torch.cuda.Stream()
    for splits, teams in ((1, 1), (2, 1), (4, 1), (8, 1), (8, 2), (8, 4), (8, 8), (4, 8), (1, 32)):
        if splits * teams * 2 > keys // 64 + 1:
            continue
        launches = {"mma": lambda: K.attention_decode(fused, k_pool, v_pool, batch, rope, None, kv, qpk, d, scale, 0, hpk,
                                                      warps, splits, key_split=key_split, n_teams=teams)}
        if K.attention_decode_tc_supports(d, qpk):
            launches["tcgen05"] = lambda: K.attention_decode_tc(fused, k_pool, v_pool, batch, rope, kv, qpk, d, scale,
                                                                splits, n_teams=teams)
        for name, launch in launches.items():
            with torch.cuda.stream(side):
                for _ in range(3):
                    launch()
                graph = torch.cuda.CUDAGraph()
                with NoCollection(), torch.cuda.graph(graph, stream=side):
                    for _ in range(20):
                        launch()
                graph.replay()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                for _ in range(5):
                    graph.replay()
                t1.record()
            torch.cuda.synchronize()
            result[f"{name} {splits}x{teams}"] = round(t0.elapsed_time(t1) * 10.0, 1)
    K.check_device_errors("cuda:0")
    print(json.dumps(result))
    return 0


def run_prefill_attention(args):
    """Device time of the prompt attention kernels alone (10 launches in a CUDA graph, median of 5 replays):
    `--batch` prompts of `--prefill-tokens` tokens after `--past` cached ones, heads of `--shape`."""
    import math

    import torch

    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200 import kernels as K
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.attention import AttentionTiles
    from pytorch_transformers_b200.parts.base import CacheNeed

    torch.cuda.set_device(0)
    cfg = ptb.FalconConfig.from_dict(SHAPES[args.shape])
    kv, d, qpk, rows, new, past = cfg.kv_heads_eff, cfg.head_dim, cfg.q_per_kv, args.batch, args.prefill_tokens, args.past
    heads = kv * qpk
    cache = Cache([(0, CacheNeed("full", kv, d, 0), None)], rows * (past + new + 64), torch.bfloat16, "cuda")
    slots = [cache.open() for _ in range(rows)]
    for slot in slots:
        if past:
            cache.reserve(slot, past)
            cache.commit(slot, past)
    ctx = StepContext(cache, slots, [[0] * new] * rows, 1, [[]] * rows, (AttentionTiles(K),))
    k_pool, v_pool, group = cache.entry_storage(0)
    k_pool.normal_()
    v_pool.normal_()
    tiles, batch = ctx.plan(AttentionTiles.plan_key), ctx.batch_c[group]
    q = torch.randn(rows * new, heads, d, device="cuda", dtype=torch.bfloat16)
    scale = 1 / math.sqrt(d)
    flops = 0.0     # causal: token t of a prompt sees past + t + 1 keys, two products of 2 * d flops per key and head
    flops = rows * heads * 4.0 * d * (new * past + new * (new + 1) / 2)
    result = {"only": "prefill-attention", "shape": args.shape, "batch": rows, "tokens": new, "past": past,
              "GFLOP": round(flops / 1e9, 1)}
    launches = {}
    if tiles.facts["mma_tokens"] == K.TC_TILE_TOKENS and K.attention_tc_supports(d):
        launches["tcgen05"] = lambda: K.attention_tc(q, k_pool, v_pool, batch, tiles.dev["mtile_seq"], tiles.dev["mtile_q0"],
                                                     tiles.facts["n_mma_tiles"], kv, scale, None)
    if "tcgen05" in launches and d == 128 and qpk >= 2:
        def single():
            K.attention_tc_pairs(0)
            try:
                return launches["tcgen05"]()
            finally:
                K.attention_tc_pairs(1)
        launches["tcgen05, a head a block"] = single
    if K.attention_mma_supports(d) and tiles.facts["mma_tokens"] > 1:
        tokens = tiles.facts["mma_tokens"]
        hpk = max(1, min(qpk, 128 // tokens))
        launches["mma"] = lambda: K.attention_mma(q, k_pool, v_pool, batch, tiles.dev["mtile_seq"], tiles.dev["mtile_q0"],
                                                  tiles.facts["n_mma_tiles"], None, kv, scale, 0, tokens, hpk, 8, 1)
    side = torch.cuda.Stream()
    for name, launch in launches.items():
        # 10 launches in a CUDA graph: the host's work for a launch is out of the time
        with torch.cuda.stream(side):
            for _ in range(3):
                launch()
            graph = torch.cuda.CUDAGraph()
            with NoCollection(), torch.cuda.graph(graph, stream=side):
                for _ in range(10):
                    launch()
            graph.replay()
            times = []
            for _ in range(5):
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                graph.replay()
                t1.record()
                t1.synchronize()
                times.append(t0.elapsed_time(t1) * 100.0)    # ms for 10 launches -> us for one
        torch.cuda.synchronize()
        us = sorted(times)[len(times) // 2]
        result[name] = {"us": round(us, 1), "TFLOPs": round(flops / us / 1e6, 1)}
    K.check_device_errors("cuda:0")
    print(json.dumps(result))
    return 0


def run_mma_cadence(args):
    """Clocks per tcgen05.mma (M = 128, K = 16) for several N, issued back to back by one thread a block on
    operands that are already in shared or tensor memory: one block alone, and two blocks on every SM."""
    import torch

    from pytorch_transformers_b200 import kernels as K

    torch.cuda.set_device(0)
    sms = K.sm_count("cuda:0")
    result = {"only": "mma-cadence", "unit": "clocks per instruction", "reps": 4000}
    for name, tmem, blocks in (("smem A, one block", False, 1), ("tmem A, one block", True, 1),
                               ("smem A, two blocks an SM", False, 2 * sms), ("tmem A, two blocks an SM", True, 2 * sms)):
        row = {}
        for n in (16, 32, 64, 128, 256):
            if tmem and n > 128:
                continue
            K.selftest_mma_cadence("cuda:0", n, 50, tmem, blocks)     # warm-up
            row[str(n)] = round(K.selftest_mma_cadence("cuda:0", n, 1000, tmem, blocks), 1)
        result[name] = row
    K.check_device_errors("cuda:0")
    print(json.dumps(result))
    return 0


def prefill_flops_ragged(c, layers, lengths):
    """Flops of one ragged prefill of prompts of the given lengths (logits for each prompt's last token)."""
    h, nh, kvh, d, f, v = shape_sizes(c)
    total = sum(lengths)
    gemm = 2 * total * layers * ((nh + 2 * kvh) * d * h + h * h + 2 * f * h)
    attn = sum(layers * nh * 2 * 2 * d * n * (n + 1) / 2 for n in lengths)
    return gemm + attn + len(lengths) * 2 * v * h


# BASELINE's runs of the two larger shapes: prompts of seeded uniform lengths in one generate() call
BASELINE_RUNS = {"11b": {"prompts": 8, "shortest": 512, "longest": 8192, "steps": 128},
                 "40b": {"prompts": 16, "shortest": 64, "longest": 2048, "steps": 256}}


def run_config(args, model, cfg, layers, pk):
    """`--only config --shape 11b|40b`: the run that BASELINE names for the shape, through generate():
    prompts of unequal lengths in one ragged prefill (fed in steps of at most 16,384 tokens), then one
    token each for the given number of steps. Device time from CUDA events recorded as each step's tokens
    reach the host; bytes of a decode step from the lengths the sequences really have at mid-run."""
    import torch
    run = BASELINE_RUNS[args.shape]
    gen = torch.Generator().manual_seed(0)
    n, steps = run["prompts"], args.decode_steps or run["steps"]
    lengths = torch.randint(run["shortest"], run["longest"] + 1, (n,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (length,), generator=gen).tolist() for length in lengths]
    marks = []

    def on_token(r, tok):
        if r == n - 1:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append((ev, time.perf_counter()))

    def once():
        marks.clear()
        torch.cuda.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        start.record()
        t0 = time.perf_counter()
        model.generate(prompts, max_new_tokens=steps, eos_token_id=None, max_batch_size=n, on_token=on_token)
        torch.cuda.synchronize()
        return start, t0

    once()                      # sizes the cache, captures the graphs of the decode steps
    with ClockSampler() as sampler:
        start, t0 = once()
    prefill_ms = start.elapsed_time(marks[0][0])
    decode_ms = marks[0][0].elapsed_time(marks[-1][0]) / (len(marks) - 1)
    wall_ms = (marks[-1][1] - marks[0][1]) / (len(marks) - 1) * 1e3
    shape = SHAPES[args.shape]
    h, nh, kvh, d, f, v = shape_sizes(shape)
    params, _ = falcon_param_count(shape, layers)
    mid = sum(lengths) + n * (1 + steps / 2)                       # cached tokens at the middle step
    step_bytes = 2 * params + mid * layers * 2 * kvh * d * 2
    flops = prefill_flops_ragged(shape, layers, lengths)
    print(json.dumps({
        "only": "config", "shape": args.shape, "layers": layers, "layers_of_config": shape["num_hidden_layers"],
        "prompts": n, "prompt_lengths": lengths, "prompt_tokens": sum(lengths), "decode_steps": steps,
        "decode": {"tokens_per_s": round(n / decode_ms * 1e3, 1), "ms_per_step": round(decode_ms, 4),
                   "ms_per_step_wall": round(wall_ms, 4), "bytes_per_step": int(step_bytes),
                   "achieved_GBps": round(step_bytes / decode_ms / 1e6, 1),
                   "frac": round(step_bytes / decode_ms / 1e6 / pk["hbm_gbs"], 4)},
        "prefill": {"tokens_per_s": round(sum(lengths) / prefill_ms * 1e3, 1), "ms": round(prefill_ms, 2),
                    "TFLOPs": round(flops / prefill_ms / 1e9, 1),
                    "frac": round(flops / prefill_ms / 1e9 / pk["bf16_tflops"], 4),
                    "frac_sustained": round(flops / prefill_ms / 1e9 / pk["bf16_tflops_sustained"], 4)},
        "peaks": pk["source"], "clocks": sampler.summary()}))
    return 0


def run_linear(args):
    """`--only linear --rows R`: device time of one linear layer of `--shape` at R rows, for the three ways
    the library has of running it: the weight-streaming kernel (up to 32 rows), the library product
    (cuBLAS through torch) and the tcgen05 kernel (up to 128 rows). 20 launches in a CUDA graph go round
    enough copies of the matrix that every launch reads its weights from HBM, not from L2."""
    import torch

    from pytorch_transformers_b200 import kernels as K

    torch.cuda.set_device(0)
    h, nh, kvh, d, f, v = shape_sizes(SHAPES[args.shape])
    rows = args.rows
    shapes = {"qkv": ((nh + 2 * kvh) * d, h), "out": (h, nh * d), "up": (f, h), "down": (h, f), "head": (v, h)}
    x_cache = {}
    result = {"only": "linear", "shape": args.shape, "rows": rows, "unit": "us per launch (GB/s of the matrix)"}
    side = torch.cuda.Stream()
    for name, (n, k) in shapes.items():
        copies = max(2, -(-(300 << 20) // (n * k * 2)))
        ws = [torch.randn(n, k, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = x_cache.setdefault(k, torch.randn(rows, k, device="cuda", dtype=torch.bfloat16))
        ways = {"library": lambda w: K.matmul_nt(x, w)}
        if K.skinny_linear_takes(rows, k):
            ways["skinny"] = lambda w: K.skinny_linear(x, w)
        if K.tc_linear_takes(rows, k):
            ways["tcgen05"] = lambda w: K.tc_linear(x, w)
        for way, launch in ways.items():
            with torch.cuda.stream(side):
                for i in range(3):
                    launch(ws[i % copies])
                graph = torch.cuda.CUDAGraph()
                with NoCollection(), torch.cuda.graph(graph, stream=side):
                    for i in range(20):
                        launch(ws[i % copies])
                graph.replay()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                for _ in range(5):
                    graph.replay()
                t1.record()
            torch.cuda.synchronize()
            us = t0.elapsed_time(t1) * 10.0
            result[f"{name} {way}"] = [round(us, 1), round(n * k * 2 / us / 1e3)]
        del ws
        torch.cuda.empty_cache()
    K.check_device_errors("cuda:0")
    print(json.dumps(result))
    return 0


def run_fill(args):
    """`--only fill`: device time of the random-weights kernel on one matrix of `--shape`'s feed-forward
    (bfloat16 and float32) and of the whole model of `--layers` layers through from_config."""
    import torch

    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200 import kernels as K
    from pytorch_transformers_b200.weights import generator

    torch.cuda.set_device(0)
    h, nh, kvh, d, f, v = shape_sizes(SHAPES[args.shape])
    result = {"only": "fill", "shape": args.shape}
    for dtype, name in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
        out = torch.empty((f, h), dtype=dtype, device="cuda")
        key = generator.tensor_key(0, "w")
        K.fill_normal(out, key, 0.02)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(5):
            K.fill_normal(out, key, 0.02)
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / 5
        result[f"matrix {f}x{h} {name}"] = {"ms": round(ms, 3), "Gvalues_per_s": round(f * h / ms / 1e6, 1),
                                            "GBps_written": round(out.numel() * out.element_size() / ms / 1e6, 1)}
    layers = args.layers or SHAPES[args.shape]["num_hidden_layers"]
    cfg = ptb.FalconConfig.from_dict(dict(SHAPES[args.shape], num_hidden_layers=layers))
    torch.cuda.synchronize()
    t = time.perf_counter()
    model = ptb.AutoModelForCausalLM.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    torch.cuda.synchronize()
    result["model"] = {"layers": layers, "seconds": round(time.perf_counter() - t, 2),
                       "GB": round(model.weight_bytes() / 1e9, 2)}
    print(json.dumps(result))
    return 0


def run_ours(args):
    if args.only == "sample":
        return run_sample(args)
    if args.only == "decode-attention":
        return run_decode_attention(args)
    if args.only == "prefill-attention":
        return run_prefill_attention(args)
    if args.only == "mma-cadence":
        return run_mma_cadence(args)
    if args.only == "linear":
        return run_linear(args)
    if args.only == "fill":
        return run_fill(args)
    import torch

    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200 import kernels
    from pytorch_transformers_b200.config.generation import GenerationConfig
    from pytorch_transformers_b200.sampling import DeviceSelector

    torch.cuda.set_device(0)
    shape = SHAPES[args.shape]
    layers = args.layers or shape["num_hidden_layers"]
    cfg = ptb.FalconConfig.from_dict(dict(shape, num_hidden_layers=layers))
    model = ptb.AutoModelForCausalLM.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    pk = peaks()
    gen = torch.Generator().manual_seed(0)

    def prompts(n, length):
        return torch.randint(0, cfg.vocab_size, (n, length), generator=gen).tolist()

    def decode_run(batch, steps, warmup, sample_clocks=False, context=CONTEXT):
        """Prefill `batch` prompts of `context` tokens, then time `steps` decode steps."""
        CONTEXT = context
        total = CONTEXT + SETTLE_STEPS + steps + warmup + 1
        cache = model.new_cache(batch * ((total + 63) // 64 * 64))
        slots = [cache.open() for _ in range(batch)]
        opts = GenerationConfig(do_sample=False)
        sel = DeviceSelector(kernels, model.device, cfg.vocab_size, opts, max_rows=batch)
        ps = prompts(batch, CONTEXT)
        chunk = max(1, 8192 // CONTEXT)                      # prompts go in a few at a time to bound activations
        for i in range(0, batch, chunk):
            logits = model.step(cache, slots[i:i + chunk], ps[i:i + chunk], want="last")
        logits = model.step(cache, slots, [[1]] * batch, want="last")
        ids = list(range(batch))

        def one():
            # one decode step as the generation loop runs it: the selection runs on the device, meanwhile
            # the host builds the next step and launches it with the tokens still on the device, then
            # reads the tokens (steps that cannot be launched ahead wait for the tokens first)
            nonlocal logits
            pending = sel.begin(logits, ids, 0)
            model.prepare_next(cache, slots)
            ahead = model.step_ahead(cache, slots, sel.device_tokens(pending))
            toks = sel.finish(pending)
            logits = ahead if ahead is not None else model.step(cache, slots, [[t] for t in toks], want="last")

        for _ in range(SETTLE_STEPS + warmup):
            one()
        torch.cuda.synchronize()
        sampler = ClockSampler() if sample_clocks else None
        l0 = kernels.launches
        if sampler:
            sampler.__enter__()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()   # a profiler started with --profile-from-start off sees the timed steps only
        start.record()
        for _ in range(steps):
            one()
        end.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        if sampler:
            sampler.__exit__()
        ms = start.elapsed_time(end) / steps
        launches = kernels.launches - l0
        ctx_mid = CONTEXT + 1 + SETTLE_STEPS + warmup + steps / 2
        cache.close_all()
        del cache
        torch.cuda.empty_cache()
        return ms, launches, ctx_mid, (sampler.summary() if sampler else None)

    if args.no_graphs:
        model.use_graphs = False
    if args.only == "config":
        return run_config(args, model, cfg, layers, pk)
    if args.only == "decode":
        ms, launches, ctx_mid, _ = decode_run(args.batch, args.steps, args.warmup, context=args.context)
        kv_bytes = args.batch * ctx_mid * layers * 2 * cfg.kv_heads_eff * cfg.head_dim * 2
        print(json.dumps({"only": "decode", "shape": args.shape, "batch": args.batch, "context": args.context,
                          "layers": layers,
                          "ms_per_step": round(ms, 4), "launches_per_step": launches / args.steps,
                          "GBps": round((model.weight_bytes() - (0 if cfg.tie_word_embeddings else
                                                                cfg.vocab_size * cfg.hidden_size * 2) + kv_bytes)
                                        / ms / 1e6, 1)}))
        return 0

    # ---- prefill of 2,048 tokens (one prompt) ----
    n_prefill = args.prefill_tokens if args.only == "prefill" else PREFILL_TOKENS
    cache = model.new_cache(n_prefill + 64)
    p = prompts(1, n_prefill)
    times = []
    for i in range(2 + 3):
        s = cache.open()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        model.step(cache, [s], p, want="last")
        b.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(a.elapsed_time(b))
        cache.close(s)
    del cache
    pre_ms = statistics.median(times)
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "shape": args.shape, "tokens": n_prefill, "layers": layers,
                          "ms": round(pre_ms, 3),
                          "TFLOPs": round(prefill_flops(shape, layers, n_prefill) / pre_ms / 1e9, 1)}))
        return 0
    pre_flops = prefill_flops(FALCON_7B, layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / pre_ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
               "frac": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "frac_sustained": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}

    # ---- headline: decode at batch 8 ----
    batch = args.batch
    ms, launches, ctx_mid, clocks = decode_run(batch, args.steps, args.warmup, sample_clocks=True)
    value = batch / ms * 1e3
    need = decode_bytes(FALCON_7B, layers, batch, ctx_mid)
    achieved = need / (ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]}

    points, points_roofline = {}, {}
    for b in (1, 64):
        pms, _, pctx, _ = decode_run(b, max(8, args.steps // 2), 3)
        points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
        pbytes = decode_bytes(FALCON_7B, layers, b, pctx)
        points_roofline[f"decode_b{b}"] = {"ms_per_step": round(pms, 4), "bytes": int(pbytes),
                                           "achieved": round(pbytes / (pms * 1e-3) / 1e9, 1),
                                           "frac": round(pbytes / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}

    # ---- end to end through generate(): host token lists in, host token lists out ----
    # After the prefill (seconds of tensor-core work under the power cap) the device runs its first tens of
    # decode steps 5 to 10 % slower and comes back in stages; SETTLE_STEPS untimed steps come before the W
    # warm-up steps so that the K timed steps measure decoding, not the prefill's aftermath.
    n_new = SETTLE_STEPS + args.warmup + args.steps
    ps = prompts(batch, CONTEXT)
    stamps = []
    model.generate(ps, max_new_tokens=2, eos_token_id=None, max_batch_size=batch)       # sizes the cache, warms up
    t_prefill_done = [None]

    def on_token(r, tok):
        if r == batch - 1:
            stamps.append(time.perf_counter())

    torch.cuda.synchronize()
    model.generate(ps, max_new_tokens=n_new, eos_token_id=None, max_batch_size=batch, on_token=on_token)
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    # stamps[i] is taken when step i's tokens have reached the host; steps after the warm-up count
    e2e_s = (stamps[-1] - stamps[-1 - args.steps]) / args.steps
    e2e = {"value": round(batch / e2e_s, 1), "unit": "tokens/s", "settle_steps": SETTLE_STEPS,
           "h2d_bytes_per_step": int(model.last_h2d_bytes),
           "d2h_bytes_per_step": 4 * batch}

    out = {
        "metric": "decode tokens/s, Falcon-7B shape, bf16, batch 8, context 2048", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": workload_config(layers, batch),
        "notes": {"sampling": "greedy, on the device", "cache_page": 64, "decode_steps": "CUDA graphs",
                  "timing": "CUDA events around K steps", "settle_steps": SETTLE_STEPS,
                  "settle": "untimed decode steps after every prefill, before the W warm-up steps"},
        "prefill": prefill, "roofline": roofline, "points": points, "points_roofline": points_roofline, "e2e": e2e,
        "gpu_launches": launches,
        "clocks": clocks,
    }
    print(json.dumps(out), flush=True)
    return 0


def run_reference(args):
    """The reference's own FalconForCausalLM.generate (bf16, its default attention path, its
    DynamicCache) from baseline/_ref, same shapes, random weights, same metric."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "transformers")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no installed reference"}))
        return 0
    try:
        import importlib.metadata as md
        os.environ["HF_HUB_OFFLINE"] = "1"
        os.environ["TRANSFORMERS_OFFLINE"] = "1"
        sys.path.insert(0, ref)
        real = md.version
        # the reference checks two wheels' versions at import; answer with versions in its range
        md.version = lambda n: {"tokenizers": "0.21.4", "huggingface-hub": "0.30.0"}.get(
            n.lower().replace("_", "-")) or real(n)
        import torch
        from transformers import FalconConfig, FalconForCausalLM
        torch.cuda.set_device(0)
        layers = args.layers or FALCON_7B["num_hidden_layers"]
        cfg = FalconConfig(**dict(FALCON_7B, num_hidden_layers=layers))
        torch.manual_seed(0)
        with torch.device("cuda:0"):
            model = FalconForCausalLM(cfg).to(torch.bfloat16).eval()
        batch = args.batch
        ids = torch.randint(0, cfg.vocab_size, (batch, CONTEXT), generator=torch.Generator().manual_seed(0))
        pinned = ids.pin_memory()
        stamps = []

        class Stamp:
            def put(self, value):
                value.cpu() if hasattr(value, "cpu") else None
                stamps.append(time.perf_counter())

            def end(self):
                pass

        def run(n_new, streamer=None):
            dev = pinned.to("cuda:0", non_blocking=True)
            return model.generate(dev, attention_mask=torch.ones_like(dev), max_new_tokens=n_new, do_sample=False,
                                  eos_token_id=None, pad_token_id=0, streamer=streamer)

        # device-timed decode: (prefill + W+K tokens) - (prefill + W tokens), CUDA events
        def timed(n_new):
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            run(n_new)
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b)

        timed(2)
        sampler = ClockSampler()
        with sampler:
            t_short = timed(args.warmup)
            t_long = timed(args.warmup + args.steps)
        ms = (t_long - t_short) / args.steps
        # end to end: wall clock between tokens reaching the host, warm-up steps dropped
        # (generate() batch > 1 cannot stream through TextStreamer; a plain streamer object serves)
        stamps.clear()
        try:
            run(args.warmup + args.steps, streamer=Stamp())
            per = (stamps[-1] - stamps[args.warmup]) / (len(stamps) - 1 - args.warmup)
            e2e = {"value": round(batch / per, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                   "d2h_bytes_per_step": 8 * batch}
        except Exception as e:  # noqa: BLE001
            e2e = {"value": None, "unit": "tokens/s", "error": str(e)[:200]}
        out = {"metric": "decode tokens/s, Falcon-7B shape, bf16, batch 8, context 2048", "impl": "reference",
               "value": round(batch / ms * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
               "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
               "config": workload_config(layers, batch),
               "notes": {"sampling": "greedy", "attention": "sdpa (reference default)", "cache": "DynamicCache",
                         "timing": "generate(W+K) minus generate(W), CUDA events"},
               "e2e": e2e, "gpu_launches": 0, "clocks": sampler.summary()}
        print(json.dumps(out), flush=True)
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration's (0: all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="", choices=["", "decode", "prefill", "sample", "decode-attention", "prefill-attention", "config", "linear",
                             "fill", "mma-cadence"],
                    help="run one section only and print its numbers (for profilers)")
    ap.add_argument("--shape", default="7b", choices=sorted(SHAPES), help="model shape for --only decode / prefill")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="prompt length for --only prefill")
    ap.add_argument("--context", type=int, default=CONTEXT, help="cached tokens per sequence for --only decode")
    ap.add_argument("--past", type=int, default=0, help="cached tokens before the prompt for --only prefill-attention")
    ap.add_argument("--rows", type=int, default=8, help="rows of the activation for --only linear")
    ap.add_argument("--decode-steps", type=int, default=0,
                    help="decode steps of --only config (0: the number BASELINE gives for the shape)")
    ap.add_argument("--settle", type=int, default=SETTLE_STEPS,
                    help="untimed decode steps after a prefill, before the warm-up steps (0 for profiler runs)")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step itself")
    args = ap.parse_args()
    globals()["SETTLE_STEPS"] = max(0, args.settle)
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library is a single-GPU engine, --gpus {args.gpus} is not run")
        return 2
    args.warmup = max(3, args.warmup)
    if (args.shape != "7b" or args.prefill_tokens != PREFILL_TOKENS or args.context != CONTEXT) and not args.only:
        print("--shape, --context and --prefill-tokens go with --only decode / --only prefill (the headline is measured on "
              "the 7B shape with a prefill of 2,048 tokens)")
        return 2
    if args.only == "config" and args.shape not in BASELINE_RUNS:
        print("--only config runs BASELINE's configurations of the larger shapes: --shape 11b or --shape 40b")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
