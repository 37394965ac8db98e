from . import qwen3  # noqa: F401  (registers Qwen3ForCausalLM)
from .layout import ModelLayout
from .model import Model, expected_tensors

__all__ = ["ModelLayout", "Model", "expected_tensors"]
