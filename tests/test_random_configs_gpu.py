"""Random Falcon configurations under random cuttings of the work, against the plain implementation.

The fixed tiny configurations pin known corners; this draws others: head sizes 16 to 128 (64 and 128
reach the tcgen05 kernels once a prompt passes 64 tokens), old and new arrangements of the block, one to
five query heads a K/V head, ALiBi or rotation, biases, three activations, tied and untied heads, in
float32 and bfloat16. Every request is fed as a prompt of a random length (in one step or in two), then
token by token in a batch whose members end at different times, and every logit row is compared."""
import os
import random

import numpy as np
import pytest
import torch

import plain_falcon as plain
import tiny_models as tm

pytestmark = pytest.mark.gpu


def random_config(r: random.Random) -> dict:
    d = r.choice([16, 32, 48, 64, 64, 80, 128, 128])
    new = r.random() < 0.5
    cfg = dict(vocab_size=r.choice([97, 333, 1000]), num_hidden_layers=r.choice([1, 2, 3]),
               new_decoder_architecture=new, bias=r.random() < 0.4, alibi=r.random() < 0.3,
               layer_norm_epsilon=r.choice([1e-5, 1e-6]), max_position_embeddings=2048,
               ffn_hidden_size=r.choice([64, 136, 200, 320]), tie_word_embeddings=r.random() < 0.5,
               activation=r.choice(["gelu", "gelu_new", "relu"]), bos_token_id=1, eos_token_id=2,
               rope_theta=r.choice([10000.0, 500042.0]), model_type="falcon", architectures=["FalconForCausalLM"])
    if new:
        kv = r.choice([1, 2, 3])
        heads = kv * r.choice([1, 2, 3, 4, 5])
        cfg.update(num_kv_heads=kv, num_ln_in_parallel_attn=r.choice([1, 2]))
    else:
        heads = r.choice([1, 2, 3, 5, 6])
        cfg.update(multi_query=r.random() < 0.6, parallel_attn=r.random() < 0.6)
    cfg.update(num_attention_heads=heads, hidden_size=heads * d)
    return cfg


@pytest.mark.parametrize("first_seed", range(0, 60, 10))
def test_random_configurations_and_cuttings(tmp_path, first_seed):
    import pytorch_transformers_b200 as ptb
    for seed in range(first_seed, first_seed + 10):
        r = random.Random(seed)
        cfg = random_config(r)
        dtype = r.choice(["float32", "bfloat16", "bfloat16"])
        folder = tm.write_model_folder(os.path.join(str(tmp_path), f"m{seed}"), cfg, tm.make_weights(cfg, seed),
                                       bf16=(dtype == "bfloat16"))
        model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
        raw, w = plain.load_folder(folder, torch.float64)
        g = np.random.Generator(np.random.PCG64(seed))
        lengths = [int(g.integers(2, r.choice([40, 200, 700]))) for _ in range(r.choice([1, 2, 3, 5]))]
        reqs = [g.integers(0, cfg["vocab_size"], size=n).tolist() for n in lengths]
        refs = [plain.model_logits(q, raw, w) for q in reqs]
        tol = dict(atol=1e-5, rtol=1e-4)
        if dtype == "bfloat16":     # the tiny tests' allowance, or 3 % of the logits' spread where that is more
            tol = dict(atol=max(2e-2, 0.03 * float(torch.cat(refs).std())), rtol=3e-2)
        what = f"seed {seed} {dtype} {cfg}"

        def close(got, want):
            torch.testing.assert_close(got.double().cpu(), want, msg=lambda m: f"{what}: {m}", **tol)

        cache = model.new_cache(sum((n + 63) // 64 * 64 for n in lengths) + 64)
        slots = [cache.open() for _ in reqs]
        heads = [int(g.integers(1, n + 1)) for n in lengths]
        if r.random() < 0.5:        # the prompts in two steps
            mids = [int(g.integers(1, h + 1)) for h in heads]
            model.step(cache, slots, [q[:m] for q, m in zip(reqs, mids)], want="none")
            rest = [(s, q[m:h]) for s, q, m, h in zip(slots, reqs, mids, heads) if h > m]
            if rest:
                model.step(cache, [s for s, _ in rest], [t for _, t in rest], want="none")
        else:
            out, at = model.step(cache, slots, [q[:h] for q, h in zip(reqs, heads)], want="all"), 0
            for h, ref in zip(heads, refs):
                close(out[at:at + h], ref[:h])
                at += h
        pos = list(heads)
        live = [i for i in range(len(reqs)) if pos[i] < lengths[i]]
        for _ in range(40):
            if not live:
                break
            out = model.step(cache, [slots[i] for i in live], [[reqs[i][pos[i]]] for i in live], want="last")
            for row, i in enumerate(live):
                close(out[row], refs[i][pos[i]])
                pos[i] += 1
            for i in [i for i in live if pos[i] >= lengths[i]]:
                cache.close(slots[i])
            live = [i for i in live if pos[i] < lengths[i]]
        model.check_errors()
        cache.check()


@pytest.mark.parametrize("first_seed", range(100, 130, 10))
def test_greedy_generation_on_random_configurations(tmp_path, first_seed):
    """`generate` in float32 with drawn limits on the batch and on the tokens of a step, with and without a
    stop token: the new tokens are the plain implementation's, token for token (a difference is allowed only
    where the plain logits' two largest lie within 1e-4 of each other)."""
    import pytorch_transformers_b200 as ptb
    for seed in range(first_seed, first_seed + 10):
        r = random.Random(seed)
        cfg = random_config(r)
        folder = tm.write_model_folder(os.path.join(str(tmp_path), f"g{seed}"), cfg, tm.make_weights(cfg, seed))
        model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype="float32")
        raw, w = plain.load_folder(folder, torch.float64)
        g = np.random.Generator(np.random.PCG64(seed))
        prompts = [g.integers(0, cfg["vocab_size"], size=int(g.integers(1, r.choice([10, 80, 200])))).tolist()
                   for _ in range(r.choice([1, 2, 3, 5, 7]))]
        new = r.choice([1, 3, 8, 20])
        eos = [int(g.integers(0, cfg["vocab_size"]))] if r.random() < 0.5 else None
        out = model.generate(prompts, max_new_tokens=new, eos_token_id=eos, do_sample=False,
                             max_batch_size=r.choice([1, 2, 3, 64]), max_step_tokens=r.choice([16, 100, 16384]))
        for p, o in zip(prompts, out):
            got, ref = list(o)[len(p):], plain.greedy(p, raw, w, new, eos or ())
            if got != ref:
                k = next((i for i, (a, b) in enumerate(zip(got, ref)) if a != b), min(len(got), len(ref)))
                top = torch.topk(plain.model_logits(list(p) + ref[:k], raw, w)[-1], 2).values
                assert float(top[0] - top[1]) <= 1e-4, (seed, k, got, ref)
