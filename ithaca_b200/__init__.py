"""ithaca_b200: a small, whole language-model library for one B200.

Everything between a request's tokens and its next token: a typed configuration
and an architecture registry, safetensors weights by name, layers put together
from parts, a paged cache with a slot per sequence, one step function, a
generation loop with sampling, and hand-written CUDA kernels for sm_100a beside a
true 32-bit path.
"""
from .config import LlamaConfig, register_architecture, registered_architectures
from .engine import Engine, GenerationOptions, GenStats
from .sampling import SamplingOptions
from .weights import write_random_model

__all__ = ["Engine", "GenerationOptions", "GenStats", "SamplingOptions", "LlamaConfig", "register_architecture",
           "registered_architectures", "write_random_model"]
__version__ = "0.1.0"
