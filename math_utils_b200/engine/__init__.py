"""The model, its step function and the generation loop."""
from .batch import StepEntry
from .model import DecoderModel
from .runtime import Runtime

__all__ = ["DecoderModel", "Runtime", "StepEntry"]
