"""NumPy-backed stand-in for `cupy`, used ONLY by tests/golden/generate.py.

The reference imports cupy unconditionally but runs its whole CPU path on
NumPy. This module lets the unmodified reference import in a container
without CuPy or a GPU: every `cp.<name>` resolves to `numpy.<name>`,
`cp.ndarray` is a class nothing is ever an instance of, and the device
count is 0 so the reference selects its CPU code path.
Test infrastructure; never imported by the product.
"""
import numpy as _np
from numpy import *  # noqa: F401,F403
from . import cuda  # noqa: F401


class ndarray:  # never instantiated: isinstance(x, cp.ndarray) is always False
    pass


def asnumpy(a, *args, **kwargs):
    return _np.asarray(a)


def get_array_module(*args):
    return _np


def __getattr__(name):
    return getattr(_np, name)
