"""svdq-b200: the SVDQuant W4A4 linear hot path of nunchaku, hand-written for B200 (sm_100a)."""
from . import _lib

__all__ = ["_lib"]
