"""Python front-ends of the hand-written sm_100a kernels.

Each op has a CUDA path (``libpb200_kernels.so`` through ctypes) wrapped in a
``torch.autograd.Function`` and an ``*_ref`` plain-PyTorch fp32 statement of the
same math that the tests compare against. A CUDA tensor never falls back to
the reference silently: if the library is missing the call raises.
"""
from . import _lib  # noqa: F401
from .functional import (  # noqa: F401
    add_rmsnorm, gemm, l2norm, linear, rmsnorm, rope_, softcap_cross_entropy, swiglu,
)
