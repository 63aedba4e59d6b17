"""The engine: model assembly, step function and generation loop."""
from .model import CausalLM, declared_tensors, load_model, resolve_dtype
from .step import Engine, EngineConfig, StepBatch, StepContext, TokenFeed
from .generate import GenerationResult, Generator, plan_batches

__all__ = ["CausalLM", "declared_tensors", "load_model", "resolve_dtype", "Engine", "EngineConfig", "StepBatch",
           "StepContext", "TokenFeed", "GenerationResult", "Generator", "plan_batches"]
