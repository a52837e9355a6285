"""mytorch_b200: the GPT training step of MyTorch as hand-written sm_100a CUDA
behind a C ABI (include/mytorch_b200.h), with the reference's Python interface
for that path on top. There is no CPU or PyTorch fallback: without the built
shared library the import fails, and without a CUDA device every compute call
raises."""
from . import _lib
from ._lib import MTError
from .array import DeviceArray, as_device_array, stream, synchronize
from . import fused_ops

__all__ = ["DeviceArray", "as_device_array", "stream", "synchronize", "fused_ops", "MTError"]

from .tensor import Tensor, no_grad, zeros, ones, zeros_like, randn, arange
from . import nn, optim, utils, ops
from .ops import transpose, permute, chunk, concatenate, stack
from .accelerate import Accelerator, GradScaler

__all__ += ["Tensor", "no_grad", "zeros", "ones", "zeros_like", "randn", "arange", "nn", "optim", "ops",
            "transpose", "permute", "chunk", "concatenate", "stack", "Accelerator", "GradScaler"]
