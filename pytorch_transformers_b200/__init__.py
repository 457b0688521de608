"""pytorch_transformers_b200: a small model library with generation of its own for one NVIDIA
B200 (sm_100a): typed configuration and registry, safetensors weights, models put together from
parts, a paged cache, one step function, a generation loop, sampling, trace replay.
Architecture built: Falcon."""
from . import models as _models  # noqa: F401  (registers the built-in architectures)
from .cache.paged import Cache
from .cache.pool import CacheError, CacheFull
from .config import (AutoConfig, ConfigError, FalconConfig, GenerationConfig, ModelConfig, register_architecture)
from .engine.batch import StepError
from .engine.model import CausalLM
from .modeling import AutoModelForCausalLM, FalconForCausalLM, GenerateOutput, PreTrainedCausalLM
from .parts import (BuildContext, CacheNeed, ModelSpec, ParamDecl, Part, PartSpec, ScheduleEntry, StateNeed,
                    register_part)
from .weights import WeightError, init_random, load_weights, write_random_model

__version__ = "0.1.0"
