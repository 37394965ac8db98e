from .batch import Sequence, StepBatch
from .engine import DTYPES, Engine, StepError, load_model

__all__ = ["Sequence", "StepBatch", "DTYPES", "Engine", "StepError", "load_model"]
