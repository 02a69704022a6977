"""The engine: the step function over a bound model and its cache, and generation above it."""
from .engine import DTYPES, Engine, StepEntry, StepError

__all__ = ["DTYPES", "Engine", "StepEntry", "StepError"]
