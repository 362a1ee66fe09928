from .build import library_path, BuildError
from .lib import load, KernelError, KernelLibrary

__all__ = ["library_path", "BuildError", "load", "KernelError", "KernelLibrary"]
