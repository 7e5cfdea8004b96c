from .api import Engine
from .generate import GenerationOptions, GenStats, generate_loop
from .model import DecoderModel, load_model, weight_manifest
from .step import StepError, Stepper

__all__ = ["Engine", "GenerationOptions", "GenStats", "generate_loop", "DecoderModel", "load_model",
           "weight_manifest", "StepError", "Stepper"]
