"""Plain, slow Falcon: whole sequences, no cache, one function per part, CPU torch.

Written from the formulas of the reference (paths are relative to its project root;
MF = src/transformers/models/falcon/modeling_falcon.py). It shares no code with the
package under test: it parses config.json and model.safetensors itself. It was compared
once with the reference's own FalconForCausalLM on tiny random models; the script and its
outputs are under tests/golden/.

Every function takes and returns tensors of one working dtype (float64 by default, so
that differences seen against it are the tested engine's rounding alone), on the device of
the weights they are given (the CPU, or a GPU for the widths of the large models).
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Sequence

import numpy as np
import torch

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
              "I32": torch.int32, "I64": torch.int64}


# ----------------------------------------------------------------------------- files
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """safetensors layout: u64 little-endian header size, JSON header, raw tensor bytes."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        payload = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        dt = _ST_DTYPES[info["dtype"]]
        buf = bytearray(payload[lo:hi])
        if len(buf) == 0:
            out[name] = torch.empty(info["shape"], dtype=dt)
        else:
            out[name] = torch.frombuffer(buf, dtype=dt).reshape(info["shape"]).clone()
    return out


def load_folder(folder: str, dtype=torch.float64):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights = {k: v.to(dtype) for k, v in read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    return cfg, weights


def resolve(cfg: dict) -> dict:
    """Defaults as FalconConfig.__init__ resolves them
    (src/transformers/models/falcon/configuration_falcon.py:144-200) and the layer
    constructor does for num_ln_in_parallel_attn (MF:599-600)."""
    c = dict(cfg)
    c.setdefault("num_attention_heads", 71)
    c.setdefault("hidden_size", 4544)
    c.setdefault("new_decoder_architecture", False)
    c.setdefault("multi_query", True)
    c.setdefault("parallel_attn", True)
    c.setdefault("bias", False)
    c.setdefault("alibi", False)
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rope_scaling", None)
    c.setdefault("layer_norm_epsilon", 1e-5)
    c.setdefault("activation", "gelu")
    c.setdefault("tie_word_embeddings", True)  # src/transformers/configuration_utils.py:221-223
    if c.get("num_kv_heads") is None:
        c["num_kv_heads"] = c["num_attention_heads"]
    if c.get("ffn_hidden_size") is None:
        c["ffn_hidden_size"] = 4 * c["hidden_size"]
    if c.get("num_ln_in_parallel_attn") is None and c["new_decoder_architecture"]:
        c["num_ln_in_parallel_attn"] = 2
    return c


# ----------------------------------------------------------------------------- parts
def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather, no scaling (MF:835, 896)."""
    return table[ids]


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float) -> torch.Tensor:
    """torch.nn.LayerNorm over the last axis: biased variance, affine (MF:603-612, 843)."""
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * gamma + beta


def linear(x: torch.Tensor, w: torch.Tensor, b=None) -> torch.Tensor:
    """x @ W.T, then the bias as a separate add (FalconLinear, MF:67-72)."""
    y = x @ w.T
    return y if b is None else y + b


def split_heads(fused: torch.Tensor, c: dict):
    """Fused projection [S, (nh+2G)d] -> q [S, nh, d], k and v [S, G, d] (MF:269-298).

    New architecture: groups of (q_per_kv queries, K, V) per KV head (MF:280-290);
    old multi-query: nh queries, then K, then V (MF:295-298); old multi-head: (q, k, v)
    per head (MF:291-294). Query head h uses KV head h // q_per_kv, which is what the
    reference's broadcast + flatten(2, 3) amounts to (MF:286-289).
    """
    s = fused.shape[0]
    nh = c["num_attention_heads"]
    d = c["hidden_size"] // nh
    if c["new_decoder_architecture"]:
        g = c["num_kv_heads"]
        v5 = fused.view(s, g, nh // g + 2, d)
        return v5[:, :, :-2].reshape(s, nh, d), v5[:, :, -2], v5[:, :, -1]
    if not c["multi_query"]:
        v4 = fused.view(s, nh, 3, d)
        return v4[:, :, 0], v4[:, :, 1], v4[:, :, 2]
    v3 = fused.view(s, nh + 2, d)
    return v3[:, :-2], v3[:, -2:-1], v3[:, -1:]


def rope_inv_freq(c: dict) -> torch.Tensor:
    """inv_freq_i = theta^(-2i/d) in float32 (src/transformers/modeling_rope_utils.py:67);
    'linear' scaling divides it by the factor (:100-108)."""
    d = c["hidden_size"] // c["num_attention_heads"]
    inv = 1.0 / (c["rope_theta"] ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
    sc = c.get("rope_scaling")
    if sc:
        kind = sc.get("rope_type", sc.get("type", "default"))
        if kind == "linear":
            inv = inv / sc["factor"]
        elif kind != "default":
            raise ValueError(kind)
    return inv


def rotary(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """x [S, heads, d]; angle = position * inv_freq in float32, cos/sin of cat(angle, angle)
    (MF:155-164), x*cos + rotate_half(x)*sin with rotate_half(x) = cat(-x[d/2:], x[:d/2])
    (MF:76-80, 104-107)."""
    ang = positions.float()[:, None] * inv_freq[None, :]          # float32, as the reference
    emb = torch.cat([ang, ang], -1)
    cos = emb.cos().to(x.dtype)[:, None, :]
    sin = emb.sin().to(x.dtype)[:, None, :]
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], -1)
    return x * cos + rot * sin


def alibi_slopes(nh: int) -> torch.Tensor:
    """Per-head slopes in float32 (MF:175-188)."""
    n = 2 ** math.floor(math.log2(nh))
    base = torch.tensor(2 ** (-(2 ** -(math.log2(n) - 3))), dtype=torch.float32)
    slopes = torch.pow(base, torch.arange(1, 1 + n, dtype=torch.int32))
    if n != nh:
        extra = torch.tensor(2 ** (-(2 ** -(math.log2(2 * n) - 3))), dtype=torch.float32)
        rem = min(n, nh - n)
        slopes = torch.cat([slopes, torch.pow(extra, torch.arange(1, 1 + 2 * rem, 2, dtype=torch.int32))])
    return slopes


def alibi_bias(nh: int, length: int, dtype) -> torch.Tensor:
    """[nh, length]: slope * key position, the product formed in bfloat16 (MF:196-198)."""
    pos = torch.arange(length, dtype=torch.int64)
    return (alibi_slopes(nh)[:, None].bfloat16() * pos[None, :]).to(dtype)


def attention_core(q, k, v, c: dict, bias=None) -> torch.Tensor:
    """Causal softmax((q k^T + bias) / sqrt(d)) v over one whole sequence (MF:388-393 and
    424-448; mask MF:1139-1144: key j is visible to the query at position p iff j <= p).
    q [S, nh, d]; k, v [S, G, d]; returns [S, nh*d] with heads concatenated (MF:395-397)."""
    s, nh, d = q.shape
    g = k.shape[1]
    qpk = nh // g
    out = torch.empty(s, nh, d, dtype=q.dtype, device=q.device)
    causal = torch.ones(s, s, dtype=torch.bool, device=q.device).tril()
    for h in range(nh):
        kk, vv = k[:, h // qpk], v[:, h // qpk]
        scores = q[:, h] @ kk.T
        if bias is not None:
            scores = scores + bias[h][None, :s].to(q.device)
        scores = scores / math.sqrt(d)
        scores = scores.masked_fill(~causal, float("-inf"))
        out[:, h] = torch.softmax(scores, -1) @ vv
    return out.reshape(s, nh * d)


def activation(x: torch.Tensor, name: str) -> torch.Tensor:
    """src/transformers/activations.py:59-78 (erf GELU), :49-56 (tanh form), ReLU."""
    if name == "gelu":
        return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))
    if name in ("gelu_new", "gelu_pytorch_tanh"):
        return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))
    if name == "relu":
        return torch.relu(x)
    raise ValueError(name)


def mlp(x, w: dict, prefix: str, c: dict) -> torch.Tensor:
    """dense_4h_to_h(act(dense_h_to_4h(x))) (MF:565-578)."""
    u = linear(x, w[prefix + "dense_h_to_4h.weight"], w.get(prefix + "dense_h_to_4h.bias"))
    return linear(activation(u, c["activation"]), w[prefix + "dense_4h_to_h.weight"],
                  w.get(prefix + "dense_4h_to_h.bias"))


def self_attention(x, w: dict, prefix: str, c: dict) -> torch.Tensor:
    """Fused projection, head split, position encoding, scores, output projection (MF:327-458)."""
    s = x.shape[0]
    fused = linear(x, w[prefix + "query_key_value.weight"], w.get(prefix + "query_key_value.bias"))
    q, k, v = split_heads(fused, c)
    bias = None
    if c["alibi"]:
        bias = alibi_bias(c["num_attention_heads"], s, x.dtype)
    else:
        pos = torch.arange(s, device=x.device)
        inv = rope_inv_freq(c).to(x.device)
        q, k = rotary(q, pos, inv), rotary(k, pos, inv)
    o = attention_core(q, k, v, c, bias)
    return linear(o, w[prefix + "dense.weight"], w.get(prefix + "dense.bias"))


def decoder_layer(x, w: dict, i: int, c: dict) -> torch.Tensor:
    """The four norm/residual arrangements of FalconDecoderLayer.forward (MF:614-683)."""
    p = f"transformer.h.{i}."
    eps = c["layer_norm_epsilon"]

    def ln(name, t):
        return layer_norm(t, w[p + name + ".weight"], w[p + name + ".bias"], eps)

    if c["new_decoder_architecture"] and c["num_ln_in_parallel_attn"] == 2:
        a_in, m_in = ln("ln_attn", x), ln("ln_mlp", x)                       # MF:630-632
    else:
        a_in = ln("input_layernorm", x)                                      # MF:634
        m_in = a_in                                                          # MF:652-654, 661-666
    attn = self_attention(a_in, w, p + "self_attention.", c)
    residual = x
    parallel = c["new_decoder_architecture"] or c["parallel_attn"]
    if not parallel:
        residual = x + attn                                                  # MF:656-658
        m_in = ln("post_attention_layernorm", residual)                      # MF:659
    m = mlp(m_in, w, p + "mlp.", c)
    if parallel:
        m = m + attn                                                         # MF:673-674
    return residual + m                                                      # MF:676


def model_logits(ids: Sequence[int], cfg: dict, w: dict) -> torch.Tensor:
    """Logits [S, V] at every position of one whole sequence (MF:864-1011, 1185-1254)."""
    c = resolve(cfg)
    dtype = w["transformer.word_embeddings.weight"].dtype
    x = embedding(torch.as_tensor(list(ids), dtype=torch.long), w["transformer.word_embeddings.weight"])
    for i in range(c["num_hidden_layers"]):
        x = decoder_layer(x, w, i, c)
    x = layer_norm(x, w["transformer.ln_f.weight"], w["transformer.ln_f.bias"], c["layer_norm_epsilon"])
    head = w["transformer.word_embeddings.weight"] if c["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(x, head).to(dtype)                                         # no bias (MF:1168)


def greedy(ids: Sequence[int], cfg: dict, w: dict, new_tokens: int, eos: Sequence[int] = ()) -> List[int]:
    """argmax of the last position's logits, token by token (src/transformers/generation/utils.py:3279);
    the stop token is kept as the last token (stopping_criteria.py:464-467)."""
    seq = list(ids)
    out = []
    for _ in range(new_tokens):
        nxt = int(model_logits(seq, cfg, w)[-1].argmax())
        out.append(nxt)
        seq.append(nxt)
        if nxt in eos:
            break
    return out


# ----------------------------------------------------------------------------- sampling
def temperature_probs(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """softmax(logits / T) (src/transformers/generation/logits_process.py:288;
    generation/utils.py:3275)."""
    return torch.softmax(logits.double() / temperature, -1)


def top_k_filter(logits: torch.Tensor, k: int) -> torch.Tensor:
    """Keep scores >= the k-th largest, others -inf (logits_process.py:512-518)."""
    k = min(k, logits.shape[-1])
    kth = torch.topk(logits, k)[0][..., -1, None]
    return logits.masked_fill(logits < kth, float("-inf"))


def top_p_filter(logits: torch.Tensor, p: float, min_keep: int = 1) -> torch.Tensor:
    """Ascending sort, cumulative softmax, drop the prefix whose mass is <= 1-p
    (logits_process.py:453-465)."""
    srt, idx = torch.sort(logits, descending=False)
    cum = srt.softmax(-1).cumsum(-1)
    remove = cum <= (1 - p)
    remove[..., -min_keep:] = False
    mask = remove.scatter(-1, idx, remove)
    return logits.masked_fill(mask, float("-inf"))


def repetition_penalty(logits: torch.Tensor, seen: Sequence[int], penalty: float) -> torch.Tensor:
    """Seen tokens: negative scores times the penalty, positive ones divided by it
    (logits_process.py:335-343)."""
    out = logits.clone()
    idx = torch.as_tensor(sorted(set(seen)), dtype=torch.long)
    s = out[idx]
    out[idx] = torch.where(s < 0, s * penalty, s / penalty)
    return out


def to_numpy(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float32).cpu().numpy()
