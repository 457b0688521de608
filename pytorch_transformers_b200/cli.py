"""Command line in the reference's manner: ``<command> [<args>]`` with sub-command classes that
register their own parsers (src/transformers/commands/transformers_cli.py:28-55), and for
generation the option names and defaults of the reference's text-generation example
(examples/pytorch/text-generation/run_generation.py:284-333): ``--model_name_or_path --prompt
--length --stop_token --temperature --repetition_penalty --k --p --seed --num_return_sequences``.
That script always samples (:408-417); ``--greedy`` is ours. Prompts are token ids
(``--prompt_ids 5,17,3``, repeatable); ``--prompt TEXT`` works when the model folder has a
tokenizer.json and the ``tokenizers`` wheel is importable.

    python -m pytorch_transformers_b200.cli run-generation --model_name_or_path DIR --prompt_ids 1,2,3
    python -m pytorch_transformers_b200.cli random-model --config config.json --seed 0 --out DIR
    python -m pytorch_transformers_b200.cli replay --model DIR --dtype float32 --out DIR --max-tokens N < steps
    python -m pytorch_transformers_b200.cli env
    python -m pytorch_transformers_b200.cli bench -- --steps 20
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional


class BaseCommand:
    @staticmethod
    def register_subcommand(sub) -> None:
        raise NotImplementedError

    def run(self) -> int:
        raise NotImplementedError


def _load_tokenizer(folder: str):
    path = os.path.join(folder, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(path)


class RunGenerationCommand(BaseCommand):
    @staticmethod
    def register_subcommand(sub) -> None:
        p = sub.add_parser("run-generation", help="generate continuations of prompts")
        p.add_argument("--model_type", default=None, help="checked against config.json if given (e.g. falcon)")
        p.add_argument("--model_name_or_path", required=True, help="model folder (config.json + safetensors)")
        p.add_argument("--prompt", type=str, default="", help="text prompt (needs tokenizer.json in the folder)")
        p.add_argument("--prompt_ids", action="append", default=[], help="comma-separated token ids; repeatable")
        p.add_argument("--prompts_file", default=None, help="JSON file with a list of token-id lists")
        p.add_argument("--length", type=int, default=20, help="new tokens per prompt")
        p.add_argument("--stop_token", type=str, default=None, help="token id (or text) at which generation stops")
        p.add_argument("--temperature", type=float, default=1.0)
        p.add_argument("--repetition_penalty", type=float, default=1.0)
        p.add_argument("--k", type=int, default=0)
        p.add_argument("--p", type=float, default=0.9)
        p.add_argument("--seed", type=int, default=42)
        p.add_argument("--num_return_sequences", type=int, default=1)
        p.add_argument("--greedy", action="store_true", help="argmax instead of sampling")
        p.add_argument("--fp32", action="store_true", help="true 32-bit path instead of bfloat16")
        p.add_argument("--batch_size", type=int, default=64)
        p.set_defaults(func=RunGenerationCommand)

    def __init__(self, args):
        self.args = args

    def run(self) -> int:
        a = self.args
        from .modeling import AutoModelForCausalLM
        model = AutoModelForCausalLM.from_pretrained(a.model_name_or_path, dtype="float32" if a.fp32 else "bfloat16")
        if a.model_type and a.model_type != model.config.model_type:
            raise SystemExit(f"--model_type {a.model_type} but the folder holds a {model.config.model_type} model")
        tok = _load_tokenizer(a.model_name_or_path)
        prompts: List[List[int]] = [[int(t) for t in s.split(",") if t.strip()] for s in a.prompt_ids]
        if a.prompts_file:
            prompts += [list(map(int, p)) for p in json.load(open(a.prompts_file))]
        if a.prompt:
            if tok is None:
                raise SystemExit("--prompt needs tokenizer.json in the model folder and the tokenizers wheel; "
                                 "give token ids with --prompt_ids instead")
            prompts.append(tok.encode(a.prompt).ids)
        if not prompts:
            bos = getattr(model.config, "bos_token_id", None)
            if bos is None:
                raise SystemExit("no prompt given (--prompt_ids, --prompts_file or --prompt)")
            prompts = [[bos]]
        eos = None
        if a.stop_token is not None:
            if a.stop_token.lstrip("-").isdigit():
                eos = int(a.stop_token)
            elif tok is not None and tok.token_to_id(a.stop_token) is not None:
                eos = tok.token_to_id(a.stop_token)
            else:
                raise SystemExit(f"--stop_token {a.stop_token!r} is neither a token id nor a known token")
        kw = dict(max_new_tokens=a.length, repetition_penalty=a.repetition_penalty, eos_token_id=eos,
                  max_batch_size=a.batch_size)
        if a.greedy:
            out = model.generate(prompts, do_sample=False, **kw)
        else:
            out = model.generate(prompts, do_sample=True, temperature=a.temperature, top_k=a.k, top_p=a.p,
                                 seed=a.seed, num_return_sequences=a.num_return_sequences, **kw)
        n_ret = 1 if a.greedy else a.num_return_sequences
        for i, seq in enumerate(out):
            prompt = prompts[i // n_ret]
            rec = {"prompt": i // n_ret, "sequence": i % n_ret, "prompt_ids": prompt, "generated_ids": seq[len(prompt):]}
            if tok is not None:
                rec["text"] = tok.decode(seq)
            print(json.dumps(rec))
        return 0


class RandomModelCommand(BaseCommand):
    @staticmethod
    def register_subcommand(sub) -> None:
        p = sub.add_parser("random-model", help="write a model folder with seeded random weights")
        p.add_argument("--config", required=True, help="a config.json (or a folder that holds one)")
        p.add_argument("--seed", type=int, default=0)
        p.add_argument("--out", required=True)
        p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
        p.set_defaults(func=RandomModelCommand)

    def __init__(self, args):
        self.args = args

    def run(self) -> int:
        import torch

        from .config.registry import lookup
        from .weights.random_init import write_random_model
        path = self.args.config
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        raw = json.load(open(path))
        cfg = lookup(raw).config_cls.from_dict(raw)
        out = write_random_model(cfg, self.args.seed, self.args.out,
                                 torch.bfloat16 if self.args.dtype == "bfloat16" else torch.float32)
        print(out)
        return 0


class ReplayCommand(BaseCommand):
    @staticmethod
    def register_subcommand(sub) -> None:
        p = sub.add_parser("replay", help="feed token traces from stdin through a model and dump logits")
        p.add_argument("--model", required=True)
        p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
        p.add_argument("--out", required=True)
        p.add_argument("--max-tokens", type=int, required=True)
        p.set_defaults(func=ReplayCommand)

    def __init__(self, args):
        self.args = args

    def run(self) -> int:
        from .engine.replay import main
        a = self.args
        return main(["--model", a.model, "--dtype", a.dtype, "--out", a.out, "--max-tokens", str(a.max_tokens)])


class EnvCommand(BaseCommand):
    @staticmethod
    def register_subcommand(sub) -> None:
        p = sub.add_parser("env", help="print the environment (src/transformers/commands/env.py does the same)")
        p.set_defaults(func=EnvCommand)

    def __init__(self, args):
        self.args = args

    def run(self) -> int:
        import platform

        import torch

        from . import __version__, native
        from .config.registry import registered
        info = {"pytorch_transformers_b200": __version__, "python": platform.python_version(),
                "platform": platform.platform(), "torch": torch.__version__, "cuda available": torch.cuda.is_available(),
                "device": torch.cuda.get_device_name(0) if torch.cuda.is_available() else None,
                "nvcc flags": " ".join(native.NVCC_FLAGS), "architectures": sorted(registered())}
        for k, v in info.items():
            print(f"- {k}: {v}")
        return 0


class BenchCommand(BaseCommand):
    """Runs the repository's benchmark (bench.py beside the package) with the arguments given after
    ``bench``; the reference keeps its benchmark outside the package too (benchmark/llama.py)."""

    @staticmethod
    def register_subcommand(sub) -> None:
        p = sub.add_parser("bench", help="run bench.py of the checkout (arguments are passed on)")
        p.add_argument("bench_args", nargs=argparse.REMAINDER, help="arguments of bench.py, e.g. --steps 20")
        p.set_defaults(func=BenchCommand)

    def __init__(self, args):
        self.args = args

    @staticmethod
    def script() -> str:
        return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")

    def run(self) -> int:
        import subprocess
        path = self.script()
        if not os.path.isfile(path):
            raise SystemExit(f"bench: {path} does not exist (the benchmark lives in the source checkout, not in an "
                             "installed package)")
        rest = [a for a in self.args.bench_args if a != "--"]
        return subprocess.call([sys.executable, path] + rest)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser("pytorch_transformers_b200 CLI tool", usage="ptb200-cli <command> [<args>]")
    sub = parser.add_subparsers(help="commands")
    for cmd in (RunGenerationCommand, RandomModelCommand, ReplayCommand, EnvCommand, BenchCommand):
        cmd.register_subcommand(sub)
    return parser


def main(argv: Optional[List[str]] = None) -> int:
    parser = build_parser()
    args = parser.parse_args(argv)
    if not hasattr(args, "func"):
        parser.print_help()
        return 1
    return args.func(args).run()


if __name__ == "__main__":
    sys.exit(main())
