"""The command line on the GPU, as a user runs it: the script in bin/ as a child process on a tiny
model folder, its tokens against the plain implementation."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_falcon as plain
import tiny_models as tm

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPT = os.path.join(ROOT, "bin", "ptb200-cli")


def run(*args):
    done = subprocess.run([sys.executable, SCRIPT, *args], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    return [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]


def ids(p):
    return ",".join(map(str, p))


def test_greedy_generation_from_the_command_line(tmp_path):
    folder = tm.tiny_folder(str(tmp_path), "A")
    raw, w = plain.load_folder(folder, torch.float64)
    prompts = tm.prompts("A", (5, 11), seed=31)
    recs = run("run-generation", "--model_name_or_path", folder, "--model_type", "falcon", "--fp32", "--greedy",
               "--length", "7", "--prompt_ids", ids(prompts[0]), "--prompt_ids", ids(prompts[1]))
    assert [r["prompt_ids"] for r in recs] == prompts
    for p, r in zip(prompts, recs):
        assert r["generated_ids"] == plain.greedy(p, raw, w, 7)
    # a stop token ends a sequence, and is kept as its last token
    free = recs[0]["generated_ids"]
    stop = free[3]
    cut = run("run-generation", "--model_name_or_path", folder, "--fp32", "--greedy", "--length", "7",
              "--stop_token", str(stop), "--prompt_ids", ids(prompts[0]))
    assert cut[0]["generated_ids"] == free[:free.index(stop) + 1]


def test_sampling_options_from_the_command_line(tmp_path):
    folder = tm.tiny_folder(str(tmp_path), "A", bf16=True)
    prompt = tm.prompts("A", (9,), seed=32)[0]
    args = ("run-generation", "--model_name_or_path", folder, "--length", "6", "--k", "20", "--p", "0.95",
            "--temperature", "1.3", "--seed", "5", "--num_return_sequences", "2", "--prompt_ids", ids(prompt))
    recs = run(*args)
    assert [(r["prompt"], r["sequence"]) for r in recs] == [(0, 0), (0, 1)]
    assert all(len(r["generated_ids"]) == 6 and all(0 <= t < 512 for t in r["generated_ids"]) for r in recs)
    assert recs[0]["generated_ids"] != recs[1]["generated_ids"]       # two draws of one prompt differ
    assert run(*args) == recs                                          # and the seed fixes them
    # the model type is checked against the folder
    done = subprocess.run([sys.executable, SCRIPT, "run-generation", "--model_name_or_path", folder, "--model_type",
                           "llama", "--prompt_ids", "1"], capture_output=True, text=True, timeout=600)
    assert done.returncode != 0 and "falcon" in done.stderr
