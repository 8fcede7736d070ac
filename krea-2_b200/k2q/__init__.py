"""k2q: B200-native rotated-quant ("ConvRot") Linear path for the Krea 2 DiT.

Python host code over ``libk2q.so`` (hand-written sm_100a CUDA behind the C ABI declared in
``include/k2q.h``).  Importing the package needs neither a GPU nor the built library; calling
any op does.
"""
from . import _lib  # noqa: F401

__all__ = ["ops", "modules", "lora", "build"]
