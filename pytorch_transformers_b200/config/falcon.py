"""FalconConfig: every config.json key of the Falcon decoder family, typed and validated.

Field names and defaults follow ``FalconConfig.__init__``
(src/transformers/models/falcon/configuration_falcon.py:144-200); the old key names of
custom-code checkpoints (``n_head``, ``n_layer``, ``n_head_kv``, ``n_embed``) are accepted
as aliases the way ``convert_custom_code_checkpoint.py:35-55`` rewrites them.
Defaults that the reference resolves late, inside modules, are resolved here once:
``num_kv_heads=None -> num_attention_heads`` (configuration_falcon.py:184),
``ffn_hidden_size=None -> 4*hidden_size`` (:195-198), ``num_ln_in_parallel_attn=None -> 2``
for the new decoder architecture (modeling_falcon.py:599-600).
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict, Optional

from .base import ModelConfig, _require

_ACTIVATIONS = ("gelu", "gelu_new", "gelu_pytorch_tanh", "relu")


@dataclasses.dataclass
class FalconConfig(ModelConfig):
    model_type: ClassVar[str] = "falcon"
    aliases: ClassVar[Dict[str, str]] = {
        "n_embed": "hidden_size",
        "n_head": "num_attention_heads",
        "n_layer": "num_hidden_layers",
        "n_head_kv": "num_kv_heads",
    }

    vocab_size: int = 65024
    hidden_size: int = 4544
    num_hidden_layers: int = 32
    num_attention_heads: int = 71
    num_ln_in_parallel_attn: Optional[int] = None
    layer_norm_epsilon: float = 1e-5
    initializer_range: float = 0.02
    use_cache: bool = True
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    num_kv_heads: Optional[int] = None
    alibi: bool = False
    new_decoder_architecture: bool = False
    multi_query: bool = True
    parallel_attn: bool = True
    bias: bool = False
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    bos_token_id: Optional[int] = 11
    eos_token_id: Optional[Any] = 11
    ffn_hidden_size: Optional[int] = None
    activation: str = "gelu"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "FalconConfig":
        raw = dict(raw)
        # a custom-code checkpoint that names n_head_kv is of the new decoder architecture
        # (convert_custom_code_checkpoint.py:44-47)
        if "n_head_kv" in raw and "new_decoder_architecture" not in raw:
            raw["new_decoder_architecture"] = True
        raw.pop("auto_map", None)
        return super().from_dict(raw)  # type: ignore[return-value]

    def __post_init__(self) -> None:
        for name in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                     "max_position_embeddings"):
            value = getattr(self, name)
            _require(isinstance(value, int) and not isinstance(value, bool) and value > 0,
                     f"{name} must be a positive integer, got {value!r}")
        if self.num_kv_heads is None:
            self.num_kv_heads = self.num_attention_heads
        if self.ffn_hidden_size is None:
            self.ffn_hidden_size = 4 * self.hidden_size
        if self.new_decoder_architecture and self.num_ln_in_parallel_attn is None:
            self.num_ln_in_parallel_attn = 2
        _require(self.hidden_size % self.num_attention_heads == 0,
                 f"hidden_size must be divisible by num_attention_heads (got {self.hidden_size} and "
                 f"{self.num_attention_heads})")  # modeling_falcon.py:243-247
        _require(isinstance(self.num_kv_heads, int) and self.num_kv_heads > 0,
                 f"num_kv_heads must be a positive integer, got {self.num_kv_heads!r}")
        _require(isinstance(self.ffn_hidden_size, int) and self.ffn_hidden_size > 0,
                 f"ffn_hidden_size must be a positive integer, got {self.ffn_hidden_size!r}")
        _require(self.layer_norm_epsilon > 0, "layer_norm_epsilon must be positive")
        _require(self.activation in _ACTIVATIONS,
                 f"activation {self.activation!r} is not supported (supported: {', '.join(_ACTIVATIONS)})")
        if self.new_decoder_architecture:
            _require(self.num_ln_in_parallel_attn in (1, 2),
                     f"num_ln_in_parallel_attn must be 1 or 2, got {self.num_ln_in_parallel_attn!r}")
            _require(self.num_attention_heads % self.num_kv_heads == 0,
                     f"num_attention_heads ({self.num_attention_heads}) must be a multiple of num_kv_heads "
                     f"({self.num_kv_heads})")
        elif not self.multi_query:
            # old architecture without multi_query views the projection as [heads, 3, head_dim]
            # (modeling_falcon.py:291-294): one K and V per query head
            _require(self.num_kv_heads == self.num_attention_heads,
                     "without new_decoder_architecture and multi_query, num_kv_heads must equal "
                     f"num_attention_heads (got {self.num_kv_heads} and {self.num_attention_heads})")
        if not self.alibi:
            _require(self.head_dim % 2 == 0, f"rotary position encoding needs an even head_dim, got {self.head_dim}")
            _require(self.rope_theta > 0, "rope_theta must be positive")
        kind, factor = self.rope_scaling_kind()
        _require(kind in ("default", "linear"),
                 f"rope_scaling type {kind!r} is not supported (supported: default, linear)")
        _require(factor >= 1.0, f"rope_scaling factor must be >= 1, got {factor}")

    # ------------------------------------------------------------------ derived values
    @property
    def head_dim(self) -> int:  # configuration_falcon.py:202-204
        return self.hidden_size // self.num_attention_heads

    @property
    def rotary(self) -> bool:  # configuration_falcon.py:206-208
        return not self.alibi

    @property
    def kv_heads_eff(self) -> int:
        """K/V heads that the fused projection really holds (modeling_falcon.py:252-263)."""
        if self.new_decoder_architecture:
            return int(self.num_kv_heads)
        return 1 if self.multi_query else self.num_attention_heads

    @property
    def q_per_kv(self) -> int:
        return self.num_attention_heads // self.kv_heads_eff

    @property
    def block_variant(self) -> str:
        """Norm placement and residual form of a decoder layer (modeling_falcon.py:588-683).

        ``two_norm_parallel``: ln_attn and ln_mlp, attention and MLP side by side;
        ``one_norm_parallel``: input_layernorm feeds both; ``sequential``: input_layernorm,
        attention, post_attention_layernorm, MLP. The new decoder architecture is always
        parallel (configuration_falcon.py:64-66).
        """
        if self.new_decoder_architecture:
            return "two_norm_parallel" if self.num_ln_in_parallel_attn == 2 else "one_norm_parallel"
        return "one_norm_parallel" if self.parallel_attn else "sequential"

    def rope_scaling_kind(self):
        if not self.rope_scaling:
            return "default", 1.0
        kind = self.rope_scaling.get("rope_type", self.rope_scaling.get("type", "default"))
        factor = float(self.rope_scaling.get("factor", 1.0)) if kind != "default" else 1.0
        return kind, factor
