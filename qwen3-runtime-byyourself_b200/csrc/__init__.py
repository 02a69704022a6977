"""Hand-written CUDA for sm_100a, its build step and its Python face."""
from .build import KernelBuildError, compile_library, load_library, loaded_libraries
from .ops import KernelError

__all__ = ["KernelBuildError", "KernelError", "compile_library", "load_library", "loaded_libraries"]
