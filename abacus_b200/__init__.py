"""abacus_b200: a small model library with generation of its own for the Qwen3 dense decoder on one B200."""
__version__ = "0.1.0"

from .config import ConfigError, Qwen3Config, load_config, register_architecture  # noqa: F401
from .weights import WeightError, write_random_model  # noqa: F401


def __getattr__(name):
    # the engine needs torch.cuda and compiled kernels; import it only when asked for
    if name in ("Engine", "load_model", "StepError"):
        from . import engine
        return getattr(engine, name)
    if name in ("LM", "generate"):
        from . import api
        return getattr(api, name)
    raise AttributeError(name)
