from .engine import ContextOverflow, Engine, StepEntry
from .loading import build_model, parse_dtype

__all__ = ["ContextOverflow", "Engine", "StepEntry", "build_model", "parse_dtype"]
