from .engine import Engine, StepEntry, EngineError, EmbeddingOov, KernelWaitTimeout, parse_dtype

__all__ = ["Engine", "StepEntry", "EngineError", "EmbeddingOov", "KernelWaitTimeout", "parse_dtype"]
