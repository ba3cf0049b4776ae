from . import library, ops
from .library import KernelLibraryError
from .ops import KernelError

__all__ = ["library", "ops", "KernelLibraryError", "KernelError"]
