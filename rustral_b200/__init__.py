"""rustral_b200: a B200-native deep-learning framework with the capabilities of Rustral.

PyTorch is the tensor front end; every CUDA hot path is a hand-written sm_100a kernel bound through
ctypes (``rustral_b200._native``); CPU tensors run on the fp32 reference math that also serves as
the numerical oracle.
"""
__version__ = "0.1.0"

from . import _native  # noqa: F401
