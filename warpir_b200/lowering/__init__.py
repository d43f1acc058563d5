"""Lowering of tile programs to sm_100a (replaces the reference's ThunderKittens emitter)."""
from .lowering import Sm100Lowerer, ThunderKittensLowerer

__all__ = ["Sm100Lowerer", "ThunderKittensLowerer"]
