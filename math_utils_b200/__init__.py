"""math_utils_b200: a small GPT-2 inference library for one B200.

Typed configuration and registry (``config``), safetensors weights and a
random-weights mode (``weights``), layers put together from parts (``parts``),
a paged cache with slots (``cache``), one step function and a generation loop
(``engine``), sampling (``sampling``), and hand-written CUDA kernels for
sm_100a (``csrc``).
"""
from . import parts as _parts  # noqa: F401  (registers the part kinds)
from .config import ConfigError, Gpt2Config, load_config, register_architecture
from .engine import DecoderModel, StepEntry
from .llm import LLM, Options
from .sampling import SamplingParams
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "DecoderModel", "Gpt2Config", "LLM", "Options", "SamplingParams", "StepEntry",
           "WeightError", "load_config",
           "register_architecture", "write_random_model"]
__version__ = "0.1.0"
