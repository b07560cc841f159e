from .library import KernelError, library
from . import ops

__all__ = ["KernelError", "library", "ops"]
