from .base import ConfigError, ModelConfig
from .falcon import FalconConfig
from .generation import GenerationConfig
from .registry import AutoConfig, Architecture, lookup, lookup_config, register_architecture, registered
