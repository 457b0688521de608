"""Trace replay: feed given token ids through a model step by step and write the logits.

It samples nothing and has no forward pass, cache or loader of its own: it loads the model as
``AutoModelForCausalLM.from_pretrained`` does, makes the cache with ``new_cache`` and calls
``step``, the same objects that generation uses. Input: one JSON object per line,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` give each request's next tokens and the places among them whose logits are wanted;
``end`` names requests that are finished after the step (their slots and pages go back). For a
step that wants something, ``<out>/<step>.f32`` holds the logits [wanted, vocab] as
little-endian float32, in the order of the entries and of ``want``. After every step the line
``done <step>`` is printed and flushed. The nearest thing in the reference are its tests that
compare a prefill plus single tokens with one full pass
(tests/models/falcon/test_modeling_falcon.py:203-263).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, IO, Optional

import numpy as np


def replay(model, cache, lines, out_dir: str, log: IO = sys.stdout) -> None:
    slots: Dict[str, int] = {}
    os.makedirs(out_dir, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = rec.get("entries", [])
        if entries:
            ids, token_lists, want = [], [], []
            for e in entries:
                rid = str(e["id"])
                if rid not in slots:
                    slots[rid] = cache.open()
                ids.append(slots[rid])
                token_lists.append([int(t) for t in e["tokens"]])
                want.append([int(w) for w in e.get("want", [])])
            logits = model.step(cache, ids, token_lists, want)
            if logits.shape[0] > 0:
                arr = logits.detach().float().cpu().numpy().astype("<f4", copy=False)
                model.check_errors()
                tmp = os.path.join(out_dir, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                cache.close(slots.pop(rid))
        print(f"done {step}", file=log, flush=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token traces through a model and dump logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels and precisions of serving; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens held by live requests at one time (each rounded up to 64); sizes the cache")
    args = ap.parse_args(argv)
    print("trace_run: loading the library (kernels are compiled at first use)", file=sys.stderr, flush=True)
    from ..modeling import AutoModelForCausalLM
    from .. import native
    native.library()
    model = AutoModelForCausalLM.from_pretrained(args.model, dtype=args.dtype, device="cuda")
    cache = model.new_cache(max(args.max_tokens, 64))
    print("trace_run: ready", file=sys.stderr, flush=True)
    replay(model, cache, sys.stdin, args.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
