from . import library
from .library import KernelError, load_library
from . import ops

__all__ = ["KernelError", "library", "load_library", "ops"]
