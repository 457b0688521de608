"""Weights: the safetensors reader and writer, loading by name, the one error (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import pytorch_transformers_b200 as ptb
from pytorch_transformers_b200.weights import SafetensorsError, SafetensorsFile, WeightError, write_safetensors
import plain_falcon as plain
import tiny_models as tm


def load_cpu(folder, dtype="float32"):
    return ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype, device="cpu")


def test_reader_and_writer_round_trip(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
               "e": torch.empty(0, 4)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors.items(), metadata={"format": "pt"})
    with SafetensorsFile(path) as f:
        assert f.metadata == {"format": "pt"} and set(f.keys()) == set(tensors)
        for k, v in tensors.items():
            assert f.tensor(k).dtype == v.dtype and torch.equal(f.tensor(k), v)
    # the tests' own reader and writer agree with the package's
    mine = plain.read_safetensors(path)
    assert torch.equal(mine["b"], tensors["b"])
    tm.write_safetensors(str(tmp_path / "y.safetensors"), {"a": tensors["a"].numpy()})
    with SafetensorsFile(str(tmp_path / "y.safetensors")) as f:
        assert torch.equal(f.tensor("a"), tensors["a"])


def test_truncated_and_malformed_files(tmp_path):
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, {"a": torch.randn(64, 64)}.items())
    blob = open(path, "rb").read()
    open(path, "wb").write(blob[:len(blob) - 100])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(path)
    open(path, "wb").write(blob[:5])
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(path)
    open(path, "wb").write(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(path)
    open(path, "wb").write(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(path)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 8]}}).encode()
    open(path, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        SafetensorsFile(path)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_load_by_name(tmp_path, name):
    folder = tm.tiny_folder(str(tmp_path), name)
    m = load_cpu(folder)
    ref = tm.make_weights(tm.config_dict(name), tm.SEEDS[name])
    assert set(m.param_table()) == set(ref)
    assert torch.equal(m.embedding, torch.from_numpy(ref["transformer.word_embeddings.weight"]))
    blk = m.blocks[1]
    assert torch.equal(blk.children["mixer"].p_qkv_weight,
                       torch.from_numpy(ref["transformer.h.1.self_attention.query_key_value.weight"]))
    if m.spec.head_name is None:
        assert m.head is m.embedding
    else:
        assert torch.equal(m.head, torch.from_numpy(ref["lm_head.weight"]))


def test_precision_on_the_device(tmp_path):
    # matrices follow the model dtype; gains and biases are held in float32 whatever the file has
    m = load_cpu(tm.tiny_folder(str(tmp_path / "f"), "B"), "bfloat16")
    mixer = m.blocks[0].children["mixer"]
    assert mixer.p_qkv_weight.dtype == torch.bfloat16 and mixer.p_qkv_bias.dtype == torch.float32
    assert m.blocks[0].children["norm_mixer"].p_weight.dtype == torch.float32
    ref = tm.make_weights(tm.config_dict("B"), tm.SEEDS["B"])
    assert torch.equal(mixer.p_qkv_bias, torch.from_numpy(ref["transformer.h.0.self_attention.query_key_value.bias"]))
    m2 = load_cpu(tm.tiny_folder(str(tmp_path / "b"), "B", bf16=True), "float32")
    assert m2.blocks[0].children["mixer"].p_qkv_weight.dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = tm.config_dict("B")
    w = tm.make_weights(cfg, 1)
    del w["transformer.h.2.ln_mlp.bias"]
    del w["lm_head.weight"]
    w["transformer.h.0.mlp.dense_h_to_4h.weight"] = w["transformer.h.0.mlp.dense_h_to_4h.weight"][:, :-1]
    w["transformer.h.9.extra.weight"] = np.zeros((2, 2), np.float32)
    w["transformer.ln_f.weight"] = np.zeros((96,), np.int32)
    folder = tm.write_model_folder(str(tmp_path / "bad"), cfg, w)
    with pytest.raises(WeightError) as e:
        load_cpu(folder)
    err = e.value
    assert err.missing == ["lm_head.weight", "transformer.h.2.ln_mlp.bias"]
    assert err.unexpected == ["transformer.h.9.extra.weight"]
    assert len(err.mismatched) == 2
    msg = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shape or dtype (2)", "[320, 95]",
                  "[320, 96]", "transformer.ln_f.weight"):
        assert piece in msg


def test_names_without_prefix_stale_tables_and_tied_head(tmp_path):
    cfg = tm.config_dict("A")
    w = tm.make_weights(cfg, 0)
    bare = {k[len("transformer."):]: v for k, v in w.items()}
    bare["h.0.self_attention.rotary_emb.inv_freq"] = np.zeros(8, np.float32)
    m = load_cpu(tm.write_model_folder(str(tmp_path / "bare"), cfg, bare))
    assert torch.equal(m.embedding, torch.from_numpy(w["transformer.word_embeddings.weight"]))
    tied = dict(w)
    tied["lm_head.weight"] = w["transformer.word_embeddings.weight"].copy()
    load_cpu(tm.write_model_folder(str(tmp_path / "tied"), cfg, tied))
    tied["lm_head.weight"] = tied["lm_head.weight"] + 1
    with pytest.raises(WeightError, match="ties the head"):
        load_cpu(tm.write_model_folder(str(tmp_path / "tied_bad"), cfg, tied))


def test_sharded_checkpoint(tmp_path):
    cfg = tm.config_dict("A")
    w = tm.make_weights(cfg, 0)
    folder = str(tmp_path / "sharded")
    os.makedirs(folder)
    json.dump(cfg, open(folder + "/config.json", "w"))
    names = sorted(w)
    parts = {"model-00001-of-00002.safetensors": names[:5], "model-00002-of-00002.safetensors": names[5:]}
    for fn, ns in parts.items():
        tm.write_safetensors(os.path.join(folder, fn), {n: w[n] for n in ns}, metadata={"format": "pt"})
    json.dump({"metadata": {}, "weight_map": {n: fn for fn, ns in parts.items() for n in ns}},
              open(folder + "/model.safetensors.index.json", "w"))
    m = load_cpu(folder)
    assert torch.equal(m.embedding, torch.from_numpy(w["transformer.word_embeddings.weight"]))
    os.remove(os.path.join(folder, "model-00002-of-00002.safetensors"))
    with pytest.raises(FileNotFoundError, match="model-00002"):
        load_cpu(folder)


def test_no_weight_file(tmp_path):
    folder = str(tmp_path / "empty")
    os.makedirs(folder)
    json.dump(tm.config_dict("A"), open(folder + "/config.json", "w"))
    open(folder + "/pytorch_model.bin", "wb").write(b"x")
    with pytest.raises(FileNotFoundError, match="convert them to safetensors"):
        load_cpu(folder)


def test_random_weights_mode_writes_a_model_folder(tmp_path):
    cfg = ptb.FalconConfig.from_dict(tm.config_dict("B"))
    a = ptb.write_random_model(cfg, seed=7, folder=str(tmp_path / "a"), dtype=torch.float32)
    b = ptb.write_random_model(cfg, seed=7, folder=str(tmp_path / "b"), dtype=torch.float32)
    c = ptb.write_random_model(cfg, seed=8, folder=str(tmp_path / "c"), dtype=torch.bfloat16)
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    ca, wa = plain.load_folder(a, torch.float32)
    cb, wb = plain.load_folder(b, torch.float32)
    cc, wc = plain.load_folder(c, torch.float32)
    assert ca == cb and ptb.AutoConfig.from_pretrained(a) == cfg
    assert set(wa) == set(tm.tensor_shapes(tm.config_dict("B")))
    for k in wa:
        assert torch.equal(wa[k], wb[k]) and wa[k].shape == wc[k].shape and not torch.equal(wa[k], wc[k])
    q = wa["transformer.h.0.self_attention.query_key_value.weight"]
    assert abs(q.std().item() - 0.02) < 0.002 and abs(q.mean().item()) < 0.002
    g = wa["transformer.h.1.ln_attn.weight"]
    assert abs(g.mean().item() - 1.0) < 0.01 and g.std().item() > 0.005
    m = load_cpu(a)
    assert torch.equal(m.head, wa["lm_head.weight"])
    # plain logits exist for the written model: the folder is a complete model
    assert plain.model_logits([1, 2, 3], ca, {k: v.double() for k, v in wa.items()}).shape == (3, 1000)


def test_strict_false_only_forgives_unused_tensors(tmp_path):
    cfg = tm.config_dict("A")
    w = tm.make_weights(cfg, 0)
    w["transformer.h.0.extra.weight"] = np.zeros((2, 2), np.float32)
    folder = tm.write_model_folder(str(tmp_path / "extra"), cfg, w)
    with pytest.raises(WeightError):
        load_cpu(folder)
    import io
    import logging
    seen = io.StringIO()
    handler = logging.StreamHandler(seen)
    logging.getLogger("pytorch_transformers_b200").addHandler(handler)
    try:
        ptb.AutoModelForCausalLM.from_pretrained(folder, dtype="float32", device="cpu", strict=False)
    finally:
        logging.getLogger("pytorch_transformers_b200").removeHandler(handler)
    assert "not used by the model" in seen.getvalue() and "transformer.h.0.extra.weight" in seen.getvalue()
    del w["transformer.ln_f.bias"]
    with pytest.raises(WeightError, match="missing"):
        ptb.AutoModelForCausalLM.from_pretrained(tm.write_model_folder(str(tmp_path / "both"), cfg, w),
                                                 dtype="float32", device="cpu", strict=False)


def test_head_sizes_beyond_the_kernels_are_refused_when_the_model_is_built(tmp_path):
    cfg = ptb.FalconConfig.from_dict(tm.config_dict("A", hidden_size=1040, num_attention_heads=2))   # head size 520
    with pytest.raises(ValueError, match="head sizes from 1 to 256"):
        ptb.AutoModelForCausalLM.from_config(cfg, device="cpu", dtype="float32")


def test_without_a_dtype_the_checkpoints_own_precision_is_kept(tmp_path):
    """dtype None or "auto": config.json's torch_dtype if it names one, else what the archive stores
    (32-bit stays 32-bit; 16-bit, bfloat16 or float16, is served in bfloat16)."""
    cfg = tm.config_dict("A")
    w = tm.make_weights(cfg, 0)
    f32 = tm.write_model_folder(str(tmp_path / "f32"), cfg, w)
    bf16 = tm.write_model_folder(str(tmp_path / "bf16"), cfg, w, bf16=True)
    f16 = tm.write_model_folder(str(tmp_path / "f16"), cfg, {k: v.astype(np.float16) for k, v in w.items()})
    said = tm.write_model_folder(str(tmp_path / "said"), dict(cfg, torch_dtype="bfloat16"), w)
    load = lambda folder, **kw: ptb.AutoModelForCausalLM.from_pretrained(folder, device="cpu", **kw)
    assert load(f32).dtype == torch.float32 and load(f32, dtype="auto").embedding.dtype == torch.float32
    assert load(bf16).dtype == torch.bfloat16 and load(f16).dtype == torch.bfloat16
    assert load(said).dtype == torch.bfloat16                  # config.json's word comes first
    assert load(f32, dtype="bfloat16").dtype == torch.bfloat16 and load(bf16, torch_dtype="float32").dtype == torch.float32
    from pytorch_transformers_b200.weights.loader import checkpoint_dtype
    assert checkpoint_dtype(f32) == torch.float32 and checkpoint_dtype(f16) == torch.bfloat16
