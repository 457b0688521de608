"""The random-weights generator on the host: the NumPy implementation against the scalar restatement in
plain_random.py, the constants of the CUDA twin against the host's, slices, the law's moments,
and the model folder that the random-weights mode writes."""
import math
import os
import re

import numpy as np
import torch

import plain_random
import tiny_models as tm

from pytorch_transformers_b200.weights import generator

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_host_generator_equals_the_scalar_restatement_bit_for_bit():
    for seed, name in ((0, "transformer.word_embeddings.weight"), (7, "h.3.x"), (2 ** 40 + 5, "ü")):
        z0, z1 = generator.normal_pairs(generator.tensor_key(seed, name), 0, 300)
        for j in (0, 1, 2, 17, 150, 299):
            assert z0[j] == plain_random.standard_normal(seed, name, 2 * j)
            assert z1[j] == plain_random.standard_normal(seed, name, 2 * j + 1)
        for bf16 in (False, True):
            vals = generator.normal_values(seed, name, 3, 40, std=0.02, offset=1.0, bf16=bf16)
            for i in (0, 1, 20, 39):
                assert float(vals[i]) == plain_random.value(seed, name, 3 + i, 0.02, 1.0, bf16)


def test_far_elements_and_pairs_of_every_octant():
    # pairs far into a large tensor (indices beyond 2^32), and all eight octants of the angle
    key = generator.tensor_key(1, "big")
    first = (1 << 33) + 12345
    z0, z1 = generator.normal_pairs(key, first, 64)
    for j in range(0, 64, 7):
        assert z0[j] == plain_random.standard_normal(1, "big", 2 * (first + j))
        assert z1[j] == plain_random.standard_normal(1, "big", 2 * (first + j) + 1)
    j = np.arange(1, 65, dtype=np.uint64) + np.uint64(first)
    with np.errstate(over="ignore"):
        r = generator._mix(np.uint64(key) + j * np.uint64(generator.GAMMA))
    assert set(((r & np.uint64(0xFFFFFFFF)) >> np.uint64(29)).tolist()) == set(range(8))


def test_any_slice_can_be_regenerated_alone():
    whole = generator.normal_values(5, "w", 0, 1001)
    for first, count in ((0, 1), (1, 1), (1, 2), (2, 999), (998, 3), (17, 500)):
        assert np.array_equal(generator.normal_values(5, "w", first, count), whole[first:first + count])
    assert generator.normal_values(5, "w", 3, 0).size == 0
    assert not np.array_equal(generator.normal_values(6, "w", 0, 8), whole[:8])       # the seed matters
    assert not np.array_equal(generator.normal_values(5, "v", 0, 8), whole[:8])       # and the name


def test_values_follow_the_normal_law():
    z0, z1 = generator.normal_pairs(generator.tensor_key(0, "law"), 0, 1 << 19)
    z = np.concatenate([z0, z1])
    n = z.size
    assert abs(z.mean()) < 4 / math.sqrt(n)
    assert abs(z.var() - 1) < 4 * math.sqrt(2 / n)
    assert abs(((z - z.mean()) ** 4).mean() - 3) < 0.05
    assert abs(np.corrcoef(z0, z1)[0, 1]) < 4 / math.sqrt(n / 2)
    assert abs(np.corrcoef(z0[:-1], z0[1:])[0, 1]) < 4 / math.sqrt(n / 2)
    # the distribution function at a few points (against erf)
    for x in (-2.0, -0.5, 0.3, 1.5):
        want = 0.5 * (1 + math.erf(x / math.sqrt(2)))
        assert abs((z < x).mean() - want) < 4 * math.sqrt(want * (1 - want) / n)
    assert 4.5 < np.abs(z).max() < 6.9            # tails are there; u > 2^-33 bounds them at 6.8


def test_the_cuda_twin_holds_the_same_constants():
    src = open(os.path.join(ROOT, "pytorch_transformers_b200", "csrc", "fill_normal.cu")).read()

    def table(name):
        body = re.search(name + r"(?:\[\d+\])? = \{?([^;]*?)\}?;", src).group(1)
        return [float.fromhex(t) for t in re.findall(r"-?0x[0-9a-f.]+p[+-]?\d+", body)]

    assert table("ATANH_COEF") == list(generator.ATANH_COEF)
    assert table("SIN_COEF") == list(generator.SIN_COEF)
    assert table("COS_COEF") == list(generator.COS_COEF)
    assert table("LN2") == [generator.LN2] and table("SQRT2") == [generator.SQRT2]
    assert table("QUARTER_PI") == [generator.QUARTER_PI]
    for const in ("GAMMA", "MIX_A", "MIX_B"):
        assert f"0x{getattr(generator, const):016X}ull" in src


def test_round_to_bf16_is_torchs_rounding():
    a = generator.normal_values(3, "r", 0, 5000, std=1.0)
    a = np.concatenate([a, np.float32([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38])])
    want = torch.from_numpy(a).bfloat16().float().numpy()
    assert np.array_equal(generator.round_to_bf16(a).view(np.uint32), want.view(np.uint32))


def test_written_folder_holds_the_law(tmp_path):
    import pytorch_transformers_b200 as ptb
    import plain_falcon as plain
    for case, dtype in (("A", torch.float32), ("B", torch.bfloat16)):
        cfg = ptb.FalconConfig.from_dict(tm.config_dict(case))
        folder = ptb.write_random_model(cfg, seed=9, folder=str(tmp_path / case), dtype=dtype)
        raw, w = plain.load_folder(folder, torch.float32)
        assert set(w) == set(tm.tensor_shapes(tm.config_dict(case)))
        for name, t in w.items():
            gain = name.endswith(".weight") and t.dim() == 1
            flat = t.flatten()
            for i in (0, 1, flat.numel() // 2, flat.numel() - 1):
                assert float(flat[i]) == plain_random.value(9, name, i, 0.02, 1.0 if gain else 0.0,
                                                            dtype == torch.bfloat16), (name, i)
