"""Run the reference's own FalconForCausalLM on the tiny models, on the CPU, and save small outputs.

Usage (from the repository root; REF is the reference project's checkout):

    python tests/golden/make_golden.py REF

For each tiny configuration of tests/tiny_models.py (and the flipped block arrangements)
it builds the reference model from REF/src in float32 with its default attention path
("sdpa"; with ALiBi the "eager" path of this version adds the bias twice, once to the
scores at modeling_falcon.py:435 and once through the mask built at :1079-1085, and so
differs from the default by up to 6e-2 in these logits; the default is what is pinned),
overwrites its parameters with the tests' seeded weights, and stores in
tests/golden/<name>.npz: the token ids of one prompt, the logits at all of its positions,
and a greedy continuation. tests/test_plain.py compares tests/plain_falcon.py with these.

The reference checks the versions of two installed wheels at import
(src/transformers/dependency_versions_check.py); this script answers that check for
`tokenizers` and `huggingface-hub` with versions inside the wanted range instead of
touching the reference. Nothing of the reference is modified or copied.
"""
import importlib.metadata as md
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

CASES = {
    "A": ("A", {}), "B": ("B", {}), "C": ("C", {}), "D": ("D", {}),
    "A_sequential": ("A", {"parallel_attn": False}),
    "B_one_norm": ("B", {"num_ln_in_parallel_attn": 1}),
    "C_parallel": ("C", {"parallel_attn": True}),
}
PROMPT_LEN = {"A": 17, "B": 40, "C": 29, "D": 23}
NEW_TOKENS = 8


def main(ref_root: str) -> None:
    os.environ["HF_HUB_OFFLINE"] = "1"
    os.environ["TRANSFORMERS_OFFLINE"] = "1"
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(ref_root, "src"))
    real = md.version
    md.version = lambda n: {"tokenizers": "0.21.4", "huggingface-hub": "0.30.0"}.get(
        n.lower().replace("_", "-")) or real(n)
    import torch
    from transformers import FalconConfig, FalconForCausalLM

    import tiny_models as tm

    for case, (name, overrides) in CASES.items():
        cfg = tm.config_dict(name, **overrides)
        weights = tm.make_weights(cfg, tm.SEEDS[name])
        kwargs = {k: v for k, v in cfg.items() if k not in ("model_type", "architectures")}
        rc = FalconConfig(**kwargs)  # attention path left at the reference's default ("sdpa")
        model = FalconForCausalLM(rc).eval().float()
        sd = model.state_dict()
        used = set()
        for k in sd:
            if k == "lm_head.weight" and cfg.get("tie_word_embeddings", True):
                continue
            if k.endswith("inv_freq"):
                continue
            sd[k].copy_(torch.from_numpy(weights[k]))
            used.add(k)
        assert used == set(weights), (sorted(set(weights) - used), sorted(used - set(weights)))
        ids = tm.prompts(name, [PROMPT_LEN[name]], seed=7)[0]
        with torch.no_grad():
            t = torch.tensor([ids])
            logits = model(t).logits[0].float().numpy()
            gen = model.generate(t, max_new_tokens=NEW_TOKENS, do_sample=False, eos_token_id=None,
                                 pad_token_id=0)[0, len(ids):].tolist()
        np.savez(os.path.join(HERE, case + ".npz"), ids=np.array(ids, np.int32), logits=logits,
                 greedy=np.array(gen, np.int32))
        print(case, logits.shape, float(np.abs(logits).max()), gen)


if __name__ == "__main__":
    main(sys.argv[1])
