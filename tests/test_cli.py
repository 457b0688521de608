"""The command line: every sub-command's parser, and the sub-commands that need no GPU run for real
(random-model, env, bench's refusal of several GPUs). The reference tests its command line the
same way, through ``main`` with a patched argv (tests/utils/test_cli.py)."""
import json
import os
import subprocess
import sys

import pytest
import torch

import tiny_models as tm

import pytorch_transformers_b200 as ptb
from pytorch_transformers_b200 import cli

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_sub_command_parses_its_options():
    p = cli.build_parser()
    a = p.parse_args(["run-generation", "--model_name_or_path", "DIR", "--prompt_ids", "1,2,3", "--prompt_ids", "4",
                      "--length", "7", "--stop_token", "11", "--temperature", "0.7", "--repetition_penalty", "1.2",
                      "--k", "40", "--p", "0.8", "--seed", "3", "--num_return_sequences", "2", "--fp32"])
    assert a.func is cli.RunGenerationCommand and a.prompt_ids == ["1,2,3", "4"] and a.length == 7
    assert (a.temperature, a.repetition_penalty, a.k, a.p, a.seed, a.num_return_sequences) == (0.7, 1.2, 40, 0.8, 3, 2)
    assert a.fp32 and not a.greedy and a.stop_token == "11"
    # the defaults of the reference's example script (run_generation.py:297-321)
    d = p.parse_args(["run-generation", "--model_name_or_path", "DIR"])
    assert (d.length, d.temperature, d.repetition_penalty, d.k, d.p, d.seed, d.num_return_sequences) == \
        (20, 1.0, 1.0, 0, 0.9, 42, 1)
    a = p.parse_args(["random-model", "--config", "c.json", "--seed", "5", "--out", "OUT", "--dtype", "float32"])
    assert a.func is cli.RandomModelCommand and (a.config, a.seed, a.out, a.dtype) == ("c.json", 5, "OUT", "float32")
    a = p.parse_args(["replay", "--model", "M", "--dtype", "bfloat16", "--out", "O", "--max-tokens", "640"])
    assert a.func is cli.ReplayCommand and a.max_tokens == 640
    assert p.parse_args(["env"]).func is cli.EnvCommand
    a = p.parse_args(["bench", "--", "--steps", "20"])
    assert a.func is cli.BenchCommand and [x for x in a.bench_args if x != "--"] == ["--steps", "20"]
    with pytest.raises(SystemExit):
        p.parse_args(["run-generation"])                       # the model folder is required
    with pytest.raises(SystemExit):
        p.parse_args(["replay", "--model", "M", "--dtype", "float16", "--out", "O", "--max-tokens", "1"])


def test_no_command_prints_help_and_fails(capsys):
    assert cli.main([]) == 1
    assert "run-generation" in capsys.readouterr().out


def test_random_model_writes_the_folder_of_the_python_entry_point(tmp_path, capsys):
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tm.config_dict("B")))
    out = str(tmp_path / "cli")
    assert cli.main(["random-model", "--config", str(cfg_path), "--seed", "4", "--out", out, "--dtype", "float32"]) == 0
    assert capsys.readouterr().out.strip() == out
    cfg = ptb.FalconConfig.from_dict(tm.config_dict("B"))
    api = ptb.write_random_model(cfg, seed=4, folder=str(tmp_path / "api"), dtype=torch.float32)
    for name in ("config.json", "model.safetensors"):
        assert open(os.path.join(out, name), "rb").read() == open(os.path.join(api, name), "rb").read()
    # a folder that holds a config.json works as --config too, and the model type is found by the registry
    out2 = str(tmp_path / "cli2")
    assert cli.main(["random-model", "--config", out, "--seed", "4", "--out", out2]) == 0
    assert ptb.AutoConfig.from_pretrained(out2).num_kv_heads == 2
    model = ptb.AutoModelForCausalLM.from_pretrained(out2, dtype="float32", device="cpu")
    assert model.head.shape == (1000, 96)


def test_env_names_the_build(capsys):
    assert cli.main(["env"]) == 0
    text = capsys.readouterr().out
    assert "sm_100a" in text and "falcon" in text and "torch" in text


def test_the_script_in_bin_runs_and_bench_is_passed_on():
    script = os.path.join(ROOT, "bin", "ptb200-cli")
    done = subprocess.run([sys.executable, script, "bench", "--", "--gpus", "2"], capture_output=True, text=True,
                          timeout=120)
    assert done.returncode == 2 and "one GPU" in done.stdout
    done = subprocess.run([sys.executable, script, "run-generation", "--model_name_or_path",
                           os.path.join(ROOT, "no_such_folder")], capture_output=True, text=True, timeout=120)
    assert done.returncode != 0 and "config.json" in done.stderr
