from . import ops
from .build import KernelBuildError, build_all, compile_module, load_module

__all__ = ["ops", "KernelBuildError", "build_all", "compile_module", "load_module"]
