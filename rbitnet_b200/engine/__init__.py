from .engine import Engine, TokenizerMissing
from .generate import GenerationLoop, GenerationResult
from .model import Model
from .step import Stepper, StepEntry, StepMeta, StepContext, SeqChunk, build_meta

__all__ = ["Engine", "TokenizerMissing", "GenerationLoop", "GenerationResult", "Model", "Stepper",
           "StepEntry", "StepMeta", "StepContext", "SeqChunk", "build_meta"]
