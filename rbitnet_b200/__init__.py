"""rbitnet_b200: a small, whole text-generation library for the dense Llama decoder on one B200.

Everything between a request's token ids and its next token: typed configuration
and registry, weights by tensor name, layers put together from parts, a paged
cache with per-sequence state, one batched step function, a generation loop,
sampling, and hand-written sm_100a CUDA kernels under all of it.
"""
from . import models  # noqa: F401
from .config import LlamaConfig, load_config, register_architecture
from .engine import Engine, GenerationResult, StepEntry
from .weights import write_random_model

__all__ = ["Engine", "GenerationResult", "StepEntry", "LlamaConfig", "load_config",
           "register_architecture", "write_random_model"]
__version__ = "0.1.0"
