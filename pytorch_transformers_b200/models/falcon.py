"""Falcon as an assembly of parts: FalconConfig -> ModelSpec, with the checkpoint's tensor names.

Block arrangement per configuration (FalconDecoderLayer,
src/transformers/models/falcon/modeling_falcon.py:588-683): the new decoder architecture with
two norms (``ln_attn``, ``ln_mlp``), one shared norm (``input_layernorm``) feeding attention
and MLP side by side, or the sequential form with ``post_attention_layernorm``. Tensor names
are those of the reference's module tree (:258-261, 570-572, 594-612, 835-843, 1167-1168).
"""
from __future__ import annotations

from ..config.falcon import FalconConfig
from ..parts.base import ModelSpec, PartSpec


def _norm(cfg: FalconConfig, prefix: str) -> PartSpec:
    return PartSpec("norm", "layernorm", {"size": cfg.hidden_size, "eps": cfg.layer_norm_epsilon, "bias": True},
                    names={"weight": prefix + ".weight", "bias": prefix + ".bias"})


def _position(cfg: FalconConfig) -> PartSpec:
    if cfg.alibi:
        return PartSpec("position", "alibi", {"heads": cfg.num_attention_heads})
    _, factor = cfg.rope_scaling_kind()
    return PartSpec("position", "rotary", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta, "factor": factor})


def _linear_names(logical: str, prefix: str, bias: bool) -> dict:
    names = {logical + ".weight": prefix + ".weight"}
    if bias:
        names[logical + ".bias"] = prefix + ".bias"
    return names


def falcon_block(cfg: FalconConfig, i: int) -> PartSpec:
    p = f"transformer.h.{i}."
    mixer = PartSpec(
        "mixer", "attention",
        {"hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.kv_heads_eff,
         "head_dim": cfg.head_dim, "bias": cfg.bias},
        children={"position": _position(cfg)},
        names={**_linear_names("qkv", p + "self_attention.query_key_value", cfg.bias),
               **_linear_names("out", p + "self_attention.dense", cfg.bias)})
    ff = PartSpec(
        "feed_forward", "dense",
        {"hidden": cfg.hidden_size, "inner": cfg.ffn_hidden_size, "activation": cfg.activation, "bias": cfg.bias},
        names={**_linear_names("up", p + "mlp.dense_h_to_4h", cfg.bias),
               **_linear_names("down", p + "mlp.dense_4h_to_h", cfg.bias)})
    variant = cfg.block_variant
    if variant == "two_norm_parallel":
        children = {"norm_mixer": _norm(cfg, p + "ln_attn"), "norm_ff": _norm(cfg, p + "ln_mlp")}
        kind = "parallel"
    elif variant == "one_norm_parallel":
        children = {"norm_mixer": _norm(cfg, p + "input_layernorm")}
        kind = "parallel"
    else:
        children = {"norm_mixer": _norm(cfg, p + "input_layernorm"),
                    "norm_ff": _norm(cfg, p + "post_attention_layernorm")}
        kind = "sequential"
    children.update({"mixer": mixer, "feed_forward": ff})
    return PartSpec("block", kind, children=children)


def falcon_spec(cfg: FalconConfig) -> ModelSpec:
    return ModelSpec(
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        embedding_name="transformer.word_embeddings.weight",
        blocks=[falcon_block(cfg, i) for i in range(cfg.num_hidden_layers)],
        final_norm=_norm(cfg, "transformer.ln_f"),
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
    )


# how a checkpoint's names may differ from the model's (handled by the loader):
#   a checkpoint of the bare decoder lacks the "transformer." prefix
#   (src/transformers/modeling_utils.py:4498-4515); stale rotary tables are ignored (:4529-4532)
FALCON_NAME_RULES = {"optional_prefix": "transformer.", "ignore_suffixes": ("rotary_emb.inv_freq",)}
