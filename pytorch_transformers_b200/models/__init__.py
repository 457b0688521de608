"""Architectures: each module turns its configuration into a ModelSpec and registers itself."""
from ..config.falcon import FalconConfig
from ..config.registry import register_architecture
from .falcon import FALCON_NAME_RULES, falcon_spec

register_architecture(
    "falcon", ("FalconForCausalLM", "RWForCausalLM"), FalconConfig, falcon_spec, name_rules=FALCON_NAME_RULES,
    aliases=("RefinedWeb", "RefinedWebModel"))  # custom-code checkpoints (convert_custom_code_checkpoint.py:35-55)
