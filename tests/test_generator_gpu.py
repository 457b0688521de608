"""The fill kernel against the host generator, bit for bit, and the two ways to a random model:
filled on the device from a configuration and a seed, or written to a folder on the host and loaded."""
import numpy as np
import pytest
import torch

import tiny_models as tm

pytestmark = pytest.mark.gpu


def _bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    return t.view(torch.int16 if t.dtype == torch.bfloat16 else torch.int32).numpy()


def _host(seed, name, first, count, std, offset, dtype, bf16_values):
    from pytorch_transformers_b200.weights import generator
    v = generator.normal_values(seed, name, first, count, std, offset, bf16=bf16_values)
    return torch.from_numpy(v).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fill_kernel_equals_the_host_generator(dtype):
    from pytorch_transformers_b200 import kernels as K
    from pytorch_transformers_b200.weights import generator
    key = generator.tensor_key(4, "some.tensor")
    for count, first in ((1, 0), (2, 0), (3, 1), (1001, 7), (4096, 0), (100003, (1 << 34) + 1), (70001, 2)):
        out = torch.empty(count, dtype=dtype, device="cuda")
        K.fill_normal(out, key, 0.02, 1.0, first=first)
        want = _host(4, "some.tensor", first, count, 0.02, 1.0, dtype, dtype == torch.bfloat16)
        assert np.array_equal(_bits(out), _bits(want)), (count, first)
    # a tensor that does not start on a pair's boundary in memory
    buf = torch.zeros(1 + 999 + 1, dtype=dtype, device="cuda")
    K.fill_normal(buf[1:1000], key, 1.0, 0.0, first=0)
    assert np.array_equal(_bits(buf[1:1000]), _bits(_host(4, "some.tensor", 0, 999, 1.0, 0.0, dtype, dtype == torch.bfloat16)))
    assert float(buf[0]) == 0.0 and float(buf[-1]) == 0.0
    if dtype == torch.float32:
        out = torch.empty(5000, dtype=dtype, device="cuda")
        K.fill_normal(out, key, 0.02, 0.0, round_bf16=True)
        assert np.array_equal(_bits(out), _bits(_host(4, "some.tensor", 0, 5000, 0.02, 0.0, dtype, True)))


def _device_tensors(model):
    out = {}
    for name, (part, logical, decl) in model.param_table().items():
        if part is None:
            out[name] = model.embedding if logical == "embedding" else model.head
        else:
            out[name] = getattr(part, "p_" + logical.replace(".", "_"))
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B"])
def test_model_filled_on_the_device_equals_the_folder_written_on_the_host(tmp_path, case, dtype):
    import pytorch_transformers_b200 as ptb
    cfg = ptb.FalconConfig.from_dict(tm.config_dict(case))
    tdtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    direct = ptb.AutoModelForCausalLM.from_config(cfg, seed=3, dtype=dtype)
    folder = ptb.write_random_model(cfg, seed=3, folder=str(tmp_path / "host"), dtype=tdtype)
    loaded = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    a, b = _device_tensors(direct), _device_tensors(loaded)
    assert set(a) == set(b)
    for name in a:
        assert a[name].dtype == b[name].dtype and torch.equal(a[name], b[name]), name
    # the folder written through the device holds the same bytes
    folder2 = ptb.write_random_model(cfg, seed=3, folder=str(tmp_path / "device"), dtype=tdtype, device="cuda")
    assert open(folder + "/model.safetensors", "rb").read() == open(folder2 + "/model.safetensors", "rb").read()
    # and the models answer alike
    prompt = tm.prompts(case, (9,), seed=2)
    ca, cb = direct.new_cache(64), loaded.new_cache(64)
    assert torch.equal(direct.step(ca, [ca.open()], prompt, want="all"), loaded.step(cb, [cb.open()], prompt, want="all"))


def test_a_matrix_of_falcon_7b_equals_the_host_generator():
    from pytorch_transformers_b200 import kernels as K
    from pytorch_transformers_b200.weights import generator
    name = "transformer.h.0.mlp.dense_h_to_4h.weight"
    out = torch.empty((18176, 4544), dtype=torch.bfloat16, device="cuda")
    K.fill_normal(out, generator.tensor_key(0, name), 0.02, 0.0)
    want = _host(0, name, 0, out.numel(), 0.02, 0.0, torch.bfloat16, True).reshape(out.shape)
    assert torch.equal(out.cpu(), want)
    assert abs(float(out.float().std()) - 0.02) < 1e-4
