"""The plain implementation against outputs of the reference's own model code (tests/golden/)."""
import os

import numpy as np
import pytest
import torch

import plain_falcon as plain
import tiny_models as tm

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = {
    "A": ("A", {}), "B": ("B", {}), "C": ("C", {}), "D": ("D", {}),
    "A_sequential": ("A", {"parallel_attn": False}),
    "B_one_norm": ("B", {"num_ln_in_parallel_attn": 1}),
    "C_parallel": ("C", {"parallel_attn": True}),
}


def _weights(cfg, name, dtype):
    return {k: torch.from_numpy(v).to(dtype) for k, v in tm.make_weights(cfg, tm.SEEDS[name]).items()}


@pytest.mark.parametrize("case", sorted(CASES))
def test_plain_matches_reference_outputs(case):
    name, overrides = CASES[case]
    cfg = tm.config_dict(name, **overrides)
    gold = np.load(os.path.join(GOLDEN, case + ".npz"))
    ids = gold["ids"].tolist()
    for dtype, tol in ((torch.float32, 2e-6), (torch.float64, 2e-6)):
        logits = plain.to_numpy(plain.model_logits(ids, cfg, _weights(cfg, name, dtype)))
        assert logits.shape == gold["logits"].shape
        np.testing.assert_allclose(logits, gold["logits"], atol=tol, rtol=1e-5)
    w = _weights(cfg, name, torch.float64)
    assert plain.greedy(ids, cfg, w, len(gold["greedy"])) == gold["greedy"].tolist()


def test_plain_reads_its_own_folder(tmp_path):
    folder = tm.tiny_folder(str(tmp_path), "B")
    cfg, w = plain.load_folder(folder, torch.float32)
    ref = tm.make_weights(tm.config_dict("B"), tm.SEEDS["B"])
    assert set(w) == set(ref)
    for k in ref:
        assert np.array_equal(w[k].numpy(), ref[k])
    cfg2, wb = plain.load_folder(tm.tiny_folder(str(tmp_path / "b"), "B", bf16=True), torch.float32)
    k = "transformer.h.1.mlp.dense_h_to_4h.weight"
    assert np.array_equal(wb[k].numpy(), torch.from_numpy(ref[k]).bfloat16().float().numpy())


def test_alibi_product_is_formed_in_bfloat16():
    # head 7 of 8 has slope 2^-8: position 257 is rounded to 256 before the product
    b = plain.alibi_bias(8, 300, torch.float32)
    assert b[7, 257].item() == 1.0
    assert b[0, 299].item() == 150.0  # 0.5 * bf16(299) = 0.5 * 300
    s6 = plain.alibi_slopes(6)
    np.testing.assert_allclose(s6.numpy(), [2 ** -2, 2 ** -4, 2 ** -6, 2 ** -8, 2 ** -1, 2 ** -3], rtol=1e-6)


def test_sampling_filters():
    logits = torch.tensor([1.0, 3.0, 2.0, -1.0, 0.5])
    assert plain.top_k_filter(logits, 2).tolist() == [float("-inf"), 3.0, 2.0, float("-inf"), float("-inf")]
    kept = plain.top_p_filter(logits, 0.8)
    assert torch.isfinite(kept).tolist() == [False, True, True, False, False]
    pen = plain.repetition_penalty(logits, [0, 3], 2.0)
    assert pen.tolist() == [0.5, 3.0, 2.0, -2.0, 0.5]
