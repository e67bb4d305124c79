from .engine import ContextOverflow, Engine, StepEntry
from .loading import build_model, build_random_model, parse_dtype

__all__ = ["ContextOverflow", "Engine", "StepEntry", "build_model", "build_random_model", "parse_dtype"]
