from .batch import StepContext, StepError
from .generate import RequestResult, plan_batches, run_generation
from .model import CausalLM
