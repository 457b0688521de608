"""bin/trace_run as a user runs it: a subprocess fed steps on stdin, logits compared with the
plain implementation (float32 and bfloat16, batches of unequal lengths, slots used again)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_falcon as plain
import tiny_models as tm

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_trace(folder, dtype, steps, out, max_tokens):
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", out, "--max-tokens", str(max_tokens)],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run(tmp_path, name, dtype):
    folder = tm.tiny_folder(str(tmp_path), name, bf16=(dtype == "bfloat16"))
    cfg, w = plain.load_folder(folder, torch.float64)
    vocab = cfg["vocab_size"]
    lengths = {"a": 70, "b": 9, "c": 40, "d": 21, "e": 65}
    reqs = dict(zip(lengths, tm.prompts(name, lengths.values(), seed=21)))
    refs = {k: plain.model_logits(v, cfg, w).float().numpy() for k, v in reqs.items()}
    steps, expect = [], {}
    n = 0

    def batch(ids, decode):
        nonlocal n
        heads = {i: lengths[i] - decode[i] for i in ids}
        steps.append({"step": n, "entries": [{"id": i, "tokens": reqs[i][:heads[i]], "want": [0, heads[i] - 1]}
                                             for i in ids], "end": [i for i in ids if decode[i] == 0]})
        expect[n] = [(i, p) for i in ids for p in (0, heads[i] - 1)]
        n += 1
        live = [i for i in ids if decode[i] > 0]
        t = 0
        while live:
            ending = [i for i in live if t + 1 == decode[i]]
            steps.append({"step": n, "entries": [{"id": i, "tokens": [reqs[i][heads[i] + t]],
                                                  "want": [0] if (t % 2 == 0 or i in ending) else []} for i in live],
                          "end": ending})
            exp = [(i, heads[i] + t) for i in live if (t % 2 == 0 or i in ending)]
            if exp:
                expect[n] = exp
            n += 1
            live = [i for i in live if i not in ending]
            t += 1

    batch(["a", "b", "c"], {"a": 6, "b": 3, "c": 0})
    batch(["d", "e"], {"d": 20, "e": 32})
    out = str(tmp_path / "out")
    # the most that live requests hold, each rounded up to 64: a+b+c = 128+64+64, d+e = 64+128
    run_trace(folder, dtype, steps, out, max_tokens=256)
    tol = dict(atol=1e-5, rtol=1e-4) if dtype == "float32" else dict(atol=2e-2, rtol=3e-2)
    for step, rows in expect.items():
        got = np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, vocab)
        assert got.shape[0] == len(rows)
        for r, (i, p) in enumerate(rows):
            np.testing.assert_allclose(got[r], refs[i][p], err_msg=f"step {step} request {i} position {p}", **tol)
    assert not os.path.exists(os.path.join(out, "2.f32")) or 2 in expect
