"""Tiny Falcon configurations and seeded weights for the tests (test-side code only).

The configurations differ in every size and option: head counts and groups, sizes that
are no power of two, layers, vocabulary, eps, position encoding, biases, tying,
activation and block arrangement. Weights follow one law for all of them: matrices and
biases N(0, 0.02), LayerNorm gain 1 + N(0, 0.02), LayerNorm bias N(0, 0.02), drawn from
numpy's PCG64 so that a committed golden output can be reproduced from (config, seed).
The folder writer here is the tests' own (the package's writer is tested against it).
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict

import numpy as np

TINY = {
    # 7B-style: multi-query, one norm, parallel, rotary, tied head
    "A": dict(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
              multi_query=True, parallel_attn=True, new_decoder_architecture=False, bias=False,
              alibi=False, rope_theta=10000.0, layer_norm_epsilon=1e-5, max_position_embeddings=128,
              ffn_hidden_size=256, tie_word_embeddings=True, activation="gelu",
              bos_token_id=1, eos_token_id=2),
    # 40B-style: grouped K/V, two norms, ALiBi, biases, untied head, head size 12
    "B": dict(vocab_size=1000, hidden_size=96, num_hidden_layers=3, num_attention_heads=8,
              num_kv_heads=2, new_decoder_architecture=True, num_ln_in_parallel_attn=2,
              ffn_hidden_size=320, alibi=True, bias=True, layer_norm_epsilon=1e-6,
              max_position_embeddings=256, tie_word_embeddings=False, activation="gelu",
              bos_token_id=0, eos_token_id=7),
    # RW-style: multi-head (K/V per head), sequential block, ALiBi with a head count
    # that is no power of two (the second slope series), biases
    "C": dict(vocab_size=333, hidden_size=96, num_hidden_layers=2, num_attention_heads=6,
              multi_query=False, parallel_attn=False, new_decoder_architecture=False, bias=True,
              alibi=True, layer_norm_epsilon=3e-5, max_position_embeddings=192,
              ffn_hidden_size=200, tie_word_embeddings=True, activation="gelu",
              bos_token_id=3, eos_token_id=[5, 9]),
    # 11B-style: grouped K/V with three groups, one norm, rotary with linear scaling and a
    # large theta, head size 32, tanh GELU
    "D": dict(vocab_size=777, hidden_size=192, num_hidden_layers=4, num_attention_heads=6,
              num_kv_heads=3, new_decoder_architecture=True, num_ln_in_parallel_attn=1,
              ffn_hidden_size=136, alibi=False, bias=False, rope_theta=500042.0,
              rope_scaling={"rope_type": "linear", "factor": 2.0}, layer_norm_epsilon=1e-5,
              max_position_embeddings=512, tie_word_embeddings=True, activation="gelu_new",
              bos_token_id=11, eos_token_id=11),
    # 7B-style with the 7B's head size (64) and an odd head count: the tensor-core attention path
    "E": dict(vocab_size=400, hidden_size=192, num_hidden_layers=2, num_attention_heads=3,
              multi_query=True, parallel_attn=True, new_decoder_architecture=False, bias=False,
              alibi=False, rope_theta=10000.0, layer_norm_epsilon=1e-5, max_position_embeddings=2048,
              ffn_hidden_size=304, tie_word_embeddings=True, activation="gelu",
              bos_token_id=1, eos_token_id=2),
    # 40B-style with head size 128, grouped K/V and ALiBi on the tensor-core path
    "F": dict(vocab_size=500, hidden_size=512, num_hidden_layers=2, num_attention_heads=4,
              num_kv_heads=2, new_decoder_architecture=True, num_ln_in_parallel_attn=2,
              ffn_hidden_size=384, alibi=True, bias=True, layer_norm_epsilon=1e-5,
              max_position_embeddings=2048, tie_word_embeddings=False, activation="gelu",
              bos_token_id=0, eos_token_id=7),
    # 11B-style at head size 128: grouped K/V (4 queries per group), one norm, rotary with a large theta
    "G": dict(vocab_size=640, hidden_size=1024, num_hidden_layers=2, num_attention_heads=8,
              num_kv_heads=2, new_decoder_architecture=True, num_ln_in_parallel_attn=1,
              ffn_hidden_size=1536, alibi=False, bias=False, rope_theta=500042.0, layer_norm_epsilon=1e-5,
              max_position_embeddings=8192, tie_word_embeddings=True, activation="gelu",
              bos_token_id=11, eos_token_id=11),
}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4, "F": 5, "G": 6}


def config_dict(name: str, **overrides) -> dict:
    cfg = dict(TINY[name])
    cfg.update(overrides)
    cfg["model_type"] = "falcon"
    cfg["architectures"] = ["FalconForCausalLM"]
    return cfg


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Names and shapes as the reference saves them (module tree of
    src/transformers/models/falcon/modeling_falcon.py:258-261, 570-572, 594-612, 835-843, 1167-1168)."""
    h = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    d = h // nh
    new = cfg.get("new_decoder_architecture", False)
    mq = cfg.get("multi_query", True)
    kv = cfg.get("num_kv_heads") or nh
    g = kv if new else (1 if mq else nh)
    f = cfg.get("ffn_hidden_size") or 4 * h
    bias = cfg.get("bias", False)
    nln = cfg.get("num_ln_in_parallel_attn")
    if nln is None and new:
        nln = 2
    parallel = new or cfg.get("parallel_attn", True)
    shapes = {"transformer.word_embeddings.weight": (cfg["vocab_size"], h)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"transformer.h.{i}."
        lin = {"self_attention.query_key_value": ((nh + 2 * g) * d, h), "self_attention.dense": (h, h),
               "mlp.dense_h_to_4h": (f, h), "mlp.dense_4h_to_h": (h, f)}
        for n, s in lin.items():
            shapes[p + n + ".weight"] = s
            if bias:
                shapes[p + n + ".bias"] = (s[0],)
        if new and nln == 2:
            norms = ["ln_attn", "ln_mlp"]
        elif parallel:
            norms = ["input_layernorm"]
        else:
            norms = ["input_layernorm", "post_attention_layernorm"]
        for n in norms:
            shapes[p + n + ".weight"] = (h,)
            shapes[p + n + ".bias"] = (h,)
    shapes["transformer.ln_f.weight"] = (h,)
    shapes["transformer.ln_f.bias"] = (h,)
    if not cfg.get("tie_word_embeddings", True):
        shapes["lm_head.weight"] = (cfg["vocab_size"], h)
    return shapes


def make_weights(cfg: dict, seed: int) -> Dict[str, np.ndarray]:
    rng = np.random.Generator(np.random.PCG64(seed))
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        w = rng.standard_normal(shape).astype(np.float32) * np.float32(0.02)
        is_norm_gain = name.endswith(".weight") and len(shape) == 1
        out[name] = (w + np.float32(1.0)) if is_norm_gain else w
    return out


def write_safetensors(path: str, tensors: Dict[str, np.ndarray], metadata=None) -> None:
    codes = {np.dtype(np.float32): "F32", np.dtype(np.float16): "F16", np.dtype(np.int32): "I32",
             np.dtype(np.int64): "I64", np.dtype(np.uint16): "BF16"}
    header, blobs, off = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        b = arr.tobytes()
        header[name] = {"dtype": codes[arr.dtype], "shape": list(arr.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (round to nearest even), as uint16."""
    u = a.astype(np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def write_model_folder(folder: str, cfg: dict, weights: Dict[str, np.ndarray], bf16: bool = False) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    tensors = {k: (to_bf16_bits(v) if bf16 else v) for k, v in weights.items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
    return folder


def tiny_folder(tmp: str, name: str, bf16: bool = False, **overrides) -> str:
    cfg = config_dict(name, **overrides)
    return write_model_folder(os.path.join(tmp, f"tiny_{name}"), cfg, make_weights(cfg, SEEDS[name]), bf16=bf16)


def prompts(name: str, lengths, seed: int = 0):
    """Uniform token ids, seeded."""
    rng = np.random.Generator(np.random.PCG64(1000 + seed))
    v = TINY[name]["vocab_size"]
    return [rng.integers(0, v, size=n).tolist() for n in lengths]
