from .linear import SVDQW4A4Linear

__all__ = ["SVDQW4A4Linear"]
