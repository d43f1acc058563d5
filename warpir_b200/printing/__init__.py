"""Text form of tile programs (API of the reference's ``warpir/printing/__init__.py:1-3``)."""
from .printer import format_kernel, print_kernel

__all__ = ["print_kernel", "format_kernel"]
