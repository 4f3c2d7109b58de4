from .engine import ModelParallelEngine, ModelParallelEngineWithLMHead, ModelParallelEngineWithValueHead  # noqa: F401
