"""bench.py's command line where no GPU is needed: more than one GPU is refused with a line and exit
code 2, sizes other than the headline's need --only, and the arithmetic behind the reported fractions."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=120)


def test_more_than_one_gpu_is_refused_in_one_line():
    done = run_bench("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert done.returncode == 2
    lines = [ln for ln in done.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_other_sizes_go_with_only():
    done = run_bench("--shape", "11b")
    assert done.returncode == 2 and "--only" in done.stdout
    done = run_bench("--context", "4096")
    assert done.returncode == 2 and "--only" in done.stdout


def test_bytes_and_flops_of_the_shapes():
    sys.path.insert(0, ROOT)
    import bench
    h, f, v, layers = 4544, 18176, 65024, 32
    per_layer = h * (h + 2 * 64) + h * h + 2 * h * f           # QKV, output, up, down (no biases)
    params, one = bench.falcon_param_count(bench.FALCON_7B, layers)
    assert one == per_layer + 2 * h                             # and one norm's gain and bias
    assert params == layers * one + v * h + 2 * h               # the head's matrix once, the last norm
    # a decode step reads every weight once and the live requests' keys and values (one K/V head of 64)
    cache = 8 * 2048 * layers * 2 * 64 * 2
    assert bench.decode_bytes(bench.FALCON_7B, layers, 8, 2048) == 2 * params + cache
    # Falcon-11B: 8 K/V heads of size 128, 32 query heads
    p11, one11 = bench.falcon_param_count(bench.FALCON_11B, 60)
    assert one11 == (32 + 16) * 128 * 4096 + 4096 * 4096 + 2 * 16384 * 4096 + 2 * 4096
    assert bench.decode_bytes(bench.FALCON_11B, 60, 8, 2048) == 2 * p11 + 8 * 2048 * 60 * 2 * 8 * 128 * 2
    # Falcon-40B: two norms per layer
    _, one40 = bench.falcon_param_count(bench.FALCON_40B, 60)
    assert one40 == (128 + 16) * 64 * 8192 + 8192 * 8192 + 2 * 32768 * 8192 + 4 * 8192
    # prefill: two flops per weight and token, plus the causal attention
    flops = bench.prefill_flops(bench.FALCON_7B, layers, 2048)
    matrices = 2 * 2048 * layers * per_layer + 2 * v * h
    attention = layers * 71 * 4 * 64 * 2048 * 2049 / 2
    assert flops == matrices + attention


def test_flops_of_a_ragged_prefill_and_the_baseline_runs():
    sys.path.insert(0, ROOT)
    import bench
    # one prompt: the same count as the plain formula; several: sums over the prompts, a head row each
    assert bench.prefill_flops_ragged(bench.FALCON_7B, 32, [2048]) == bench.prefill_flops(bench.FALCON_7B, 32, 2048)
    two = bench.prefill_flops_ragged(bench.FALCON_11B, 60, [512, 8192])
    assert two == bench.prefill_flops(bench.FALCON_11B, 60, 512) + bench.prefill_flops(bench.FALCON_11B, 60, 8192)
    assert bench.BASELINE_RUNS["11b"] == {"prompts": 8, "shortest": 512, "longest": 8192, "steps": 128}
    assert bench.BASELINE_RUNS["40b"] == {"prompts": 16, "shortest": 64, "longest": 2048, "steps": 256}
    done = run_bench("--only", "config")
    assert done.returncode == 2 and "--shape 11b" in done.stdout
    # both arms describe the workload in the same words
    cfg = bench.workload_config(32, 8)
    assert len(cfg) <= 20 and all(not isinstance(v, (dict, list)) for v in cfg.values())
    assert (cfg["hidden"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["ffn"], cfg["vocab"]) == \
        (4544, 71, 1, 64, 18176, 65024)
