"""tffinfer_b200: a small, whole LLM inference engine for one B200 (sm_100a)."""
from . import log
from . import parts as _parts    # noqa: F401  registers the built-in parts
from . import models as _models  # noqa: F401  registers the architectures
from .config import EngineConfig, Qwen3Config, ConfigError
from .registry import (register_architecture, register_part, get_architecture, get_part,
                       registered_architectures, registered_parts, RegistryError)
from .weights import write_random_model, WeightError
from .engine import ModelRunner, StepEntry, OutOfPages, RequestError, Engine, InferRuntime
from .sampling import SamplingParams

__version__ = "0.1.0"
