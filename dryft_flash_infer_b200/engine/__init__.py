from .context import StepContext, StepEntry
from .engine import Engine, EngineOptions
from .generate import Request, generate_all, generate_batch
from .model import DecoderModel
from .stepper import Stepper

__all__ = ["StepContext", "StepEntry", "Engine", "EngineOptions", "Request", "generate_all", "generate_batch",
           "DecoderModel", "Stepper"]
