"""blok_b200: B200-native (sm_100a) implementation of Blok's decode hot path.

The product is the C-ABI library built from blok_b200/csrc (see include/blok_b200.h).
This package is its thin Python front end: device memory and streams come from
PyTorch, everything on the hot path runs in the CUDA library.  There is no CPU
fallback: importing the ops without the built library raises.
"""
from . import lib, synth  # noqa: F401
from .lib import BlokError, load  # noqa: F401

__all__ = ["lib", "synth", "BlokError", "load"]
