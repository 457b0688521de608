"""Configuration and registry (no GPU)."""
import json

import pytest

import pytorch_transformers_b200 as ptb
from pytorch_transformers_b200.config import ConfigError, FalconConfig, GenerationConfig
from pytorch_transformers_b200.config.registry import lookup, registered
import tiny_models as tm


def test_defaults_are_falcon_7b():
    c = FalconConfig()
    assert (c.vocab_size, c.hidden_size, c.num_hidden_layers, c.num_attention_heads) == (65024, 4544, 32, 71)
    assert c.head_dim == 64 and c.kv_heads_eff == 1 and c.q_per_kv == 71
    assert c.ffn_hidden_size == 4 * 4544 and c.num_kv_heads == 71
    assert c.block_variant == "one_norm_parallel" and c.rotary and c.tie_word_embeddings
    assert c.eos_token_ids() == (11,)


@pytest.mark.parametrize("name,variant,kv", [("A", "one_norm_parallel", 1), ("B", "two_norm_parallel", 2),
                                              ("C", "sequential", 6), ("D", "one_norm_parallel", 3)])
def test_tiny_configs_resolve(name, variant, kv):
    c = FalconConfig.from_dict(tm.config_dict(name))
    assert c.block_variant == variant and c.kv_heads_eff == kv
    again = FalconConfig.from_dict(json.loads(json.dumps(c.to_dict())))
    assert again == c


def test_new_architecture_is_always_parallel():
    c = FalconConfig.from_dict(tm.config_dict("B", parallel_attn=False))
    assert c.block_variant == "two_norm_parallel"
    c1 = FalconConfig.from_dict(tm.config_dict("B", num_ln_in_parallel_attn=1))
    assert c1.block_variant == "one_norm_parallel"


def test_old_names_of_custom_code_checkpoints():
    c = FalconConfig.from_dict({"model_type": "RefinedWeb", "n_head": 8, "n_layer": 3, "n_head_kv": 2,
                                "hidden_size": 64, "vocab_size": 100, "auto_map": {"x": "y"},
                                "architectures": ["RWForCausalLM"]})
    assert c.num_attention_heads == 8 and c.num_hidden_layers == 3 and c.num_kv_heads == 2
    assert c.new_decoder_architecture and "auto_map" not in c.extra
    assert lookup({"model_type": "RefinedWeb"}).model_type == "falcon"
    assert lookup({"architectures": ["RWForCausalLM"]}).model_type == "falcon"


def test_unknown_keys_are_kept():
    c = FalconConfig.from_dict(tm.config_dict("A", some_future_key=[1, 2]))
    assert c.extra["some_future_key"] == [1, 2] and c.to_dict()["some_future_key"] == [1, 2]


@pytest.mark.parametrize("bad", [
    dict(hidden_size=65), dict(num_attention_heads=0), dict(vocab_size=-1), dict(activation="swish"),
    dict(rope_scaling={"rope_type": "yarn", "factor": 2.0}), dict(rope_scaling={"type": "dynamic", "factor": 2.0}),
    dict(multi_query=False, num_kv_heads=2), dict(layer_norm_epsilon=0.0),
    dict(new_decoder_architecture=True, num_kv_heads=3), dict(new_decoder_architecture=True, num_ln_in_parallel_attn=3),
    dict(hidden_size=36, num_attention_heads=4),  # head_dim 9: rotary needs an even head size
])
def test_bad_values_are_refused(bad):
    with pytest.raises(ConfigError):
        FalconConfig.from_dict(tm.config_dict("A", **bad))


def test_registry(tmp_path):
    assert "falcon" in registered()
    folder = tm.tiny_folder(str(tmp_path), "A")
    assert isinstance(ptb.AutoConfig.from_pretrained(folder), FalconConfig)
    with pytest.raises(ValueError, match="Registered model types: .*falcon"):
        lookup({"model_type": "nope", "architectures": ["NopeForCausalLM"]})
    with pytest.raises(FileNotFoundError, match="config.json"):
        ptb.AutoConfig.from_pretrained(str(tmp_path / "missing"))


def test_generation_config():
    g = GenerationConfig()
    assert (g.max_length, g.do_sample, g.temperature, g.top_k, g.top_p) == (20, False, 1.0, 50, 1.0)
    assert g.new_token_budget(7) == 20 and g.new_token_budget(7, max_position_embeddings=16) == 9
    assert g.updated(max_new_tokens=5).new_token_budget(100) == 5
    assert g.updated(max_length=30).new_token_budget(12) == 18
    with pytest.raises(ValueError, match="nothing can be generated"):
        g.updated(max_length=10).new_token_budget(12)
    for bad in (dict(temperature=0.0), dict(temperature=-1), dict(top_p=0.0), dict(top_p=1.5), dict(top_k=-1),
                dict(repetition_penalty=0), dict(max_new_tokens=0), dict(num_beams=4), dict(nonsense=1),
                dict(num_return_sequences=2)):
        with pytest.raises(ValueError):
            g.updated(**bad)
    assert g.updated(eos_token_id=[3, 4]).eos_ids() == (3, 4) and g.updated(eos_token_id=7).eos_ids() == (7,)
    assert g.updated(num_beams=1, do_sample=True, num_return_sequences=2).num_return_sequences == 2


def test_generation_config_from_folder(tmp_path):
    folder = tm.tiny_folder(str(tmp_path), "C")
    cfg = ptb.AutoConfig.from_pretrained(folder)
    g = GenerationConfig.from_pretrained(folder, cfg)
    assert g.eos_ids() == (5, 9) and g.bos_token_id == 3
    with open(folder + "/generation_config.json", "w") as f:
        json.dump({"eos_token_id": 4, "max_new_tokens": 3, "do_sample": True, "temperature": 0.5,
                   "transformers_version": "4.49.0", "_from_model_config": True}, f)
    g = GenerationConfig.from_pretrained(folder, cfg)
    assert g.eos_ids() == (4,) and g.max_new_tokens == 3 and g.do_sample and g.temperature == 0.5
