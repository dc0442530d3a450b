from .engine import Engine, StepEntry, EngineError, EmbeddingOov, parse_dtype

__all__ = ["Engine", "StepEntry", "EngineError", "EmbeddingOov", "parse_dtype"]
