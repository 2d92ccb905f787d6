"""Typed configurations and the architecture registry."""
from .base import (ConfigError, KeyReader, LayerSpec, ModelPlan, PartSpec,
                   ScheduleEntry, default_schedule)
from .gpt2 import Gpt2Config
from .registry import (Architecture, architecture_for, known_architectures,
                       load_config, read_config_json, register_architecture)

register_architecture(Architecture(
    names=("gpt2", "GPT2LMHeadModel"),
    config_class=Gpt2Config,
    # some checkpoints keep every tensor under "transformer."
    name_prefixes=("", "transformer."),
), replace=True)

__all__ = [
    "Architecture", "ConfigError", "Gpt2Config", "KeyReader", "LayerSpec", "ModelPlan",
    "PartSpec", "ScheduleEntry", "architecture_for", "default_schedule",
    "known_architectures", "load_config", "read_config_json", "register_architecture",
]
