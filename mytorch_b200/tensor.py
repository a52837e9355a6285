"""Reverse-mode autograd over device arrays: the `Tensor` of the reference
(mytorch/tensor.py:26-261) thinned to what the GPT training step uses.

As in the reference, every differentiable op returns a Tensor holding a Python
closure (`grad_fn`) and its parents; `backward()` topologically sorts the graph
and runs the closures in reverse, each closure ACCUMULATING into its inputs'
`.grad` (mytorch/tensor.py:182-261). All arithmetic is done by the CUDA library;
this file only wires the graph.

Gradient dtypes: activations get gradients in their own dtype; parameters
(leaf tensors) accumulate in fp32 whatever their dtype, so several micro-batches
and the tied embedding/lm_head weight sum without half-precision loss.
"""
import numpy as np

from . import _lib
from .array import DeviceArray, as_device_array, stream

_grad_enabled = True


class no_grad:
    """Context manager disabling graph construction (mytorch/tensor.py:9-24)."""

    def __enter__(self):
        global _grad_enabled
        self._prev = _grad_enabled
        _grad_enabled = False

    def __exit__(self, *a):
        global _grad_enabled
        _grad_enabled = self._prev
        return False


def _to_device_array(data, dtype=None):
    if isinstance(data, Tensor):
        return data.data
    if isinstance(data, DeviceArray):
        return data if dtype is None else data.astype(dtype)
    if hasattr(data, "__cuda_array_interface__"):
        return as_device_array(data)
    return DeviceArray.from_numpy(np.asarray(data), dtype)


class Tensor:
    # Optional callable(param) invoked during backward() as soon as the last closure contributing to
    # a parameter's gradient has run (set by Accelerator to start that gradient's all-reduce early).
    param_ready_hook = None
    # Device scalar that loss.backward() will be called with (the loss scale of mixed-precision
    # training), announced by the Accelerator so that a loss may fold it into a gradient it
    # produces already in its forward pass. None = backward() is expected with its default of 1.
    loss_grad_hint = None
    _unit_grad_ptr = None

    def __init__(self, data, requires_grad=False, grad_fn=None, grad_fn_name=None, dtype=None, device=None):
        self.data = _to_device_array(data, dtype)
        self.requires_grad = bool(requires_grad)
        self.grad = None
        self.grad_fn = grad_fn
        self.grad_fn_name = grad_fn_name
        self._parents = ()
        self.is_param = False

    # ---- graph ----
    @staticmethod
    def build_graph_enabled():
        return _grad_enabled

    def _add_parents(self, *parents):
        self._parents = tuple(p for p in parents if isinstance(p, Tensor) and p.requires_grad)

    def backward(self, grad=None):
        """Topological sort from this tensor, closures run in reverse order;
        the graph is released afterwards (mytorch/tensor.py:182-261)."""
        if not self.requires_grad:
            raise RuntimeError("backward() on a tensor that does not require grad")
        if grad is None:
            g = DeviceArray.empty(self.shape, self.dtype).fill_(1.0)
            Tensor._unit_grad_ptr = g.ptr      # lets an op recognise "the upstream gradient is exactly 1"
        else:
            g = _to_device_array(grad, self.dtype)
            Tensor._unit_grad_ptr = None
        order, seen = [], set()
        stack = [(self, False)]
        while stack:                      # iterative DFS post-order
            node, done = stack.pop()
            if done:
                order.append(node)
                continue
            if id(node) in seen:
                continue
            seen.add(id(node))
            stack.append((node, True))
            for p in node._parents:
                if id(p) not in seen:
                    stack.append((p, False))
        self.grad = g
        exec_order = list(reversed(order))
        hook = Tensor.param_ready_hook
        last_use = {}
        if hook is not None:               # index of the last closure that writes each parameter's gradient
            for k, node in enumerate(exec_order):
                for p in node._parents:
                    if p.is_param:
                        last_use[id(p)] = (k, p)
            ready_at = {}
            for k, p in last_use.values():
                ready_at.setdefault(k, []).append(p)
        for k, node in enumerate(exec_order):
            if node.grad_fn is not None:
                node.grad_fn(node.grad)
                node.grad_fn = None
                node._parents = ()
                if not node.is_param:
                    node.grad = None      # activations' gradients are consumed
            if hook is not None:
                for p in ready_at.get(k, ()):
                    hook(p)               # every kernel writing p.grad has been queued

    def _accumulate(self, g):
        """grad += g. Takes ownership of g when there is no gradient yet."""
        if self.is_param:
            if self.grad is None:
                self.grad = DeviceArray.zeros(self.shape, "float32")
            _lib.axpby(g.ptr, 1.0, self.grad.ptr, 1.0, g.size, g.code, self.grad.code, stream())
        elif self.grad is None:
            self.grad = g
        else:
            _lib.axpby(g.ptr, 1.0, self.grad.ptr, 1.0, g.size, g.code, self.grad.code, stream())

    def param_grad_buffer(self):
        """The fp32 accumulation buffer of a parameter (created zeroed)."""
        if self.grad is None:
            self.grad = DeviceArray.zeros(self.shape, "float32")
        return self.grad

    # ---- metadata ----
    @property
    def shape(self):
        return self.data.shape

    @property
    def dtype(self):
        return self.data.dtype

    @property
    def ndim(self):
        return self.data.ndim

    @property
    def device(self):
        return "cuda"

    def numpy(self):
        return self.data.numpy()

    def item(self):
        return self.data.item()

    def __repr__(self):
        return f"Tensor(shape={self.shape}, dtype={self.dtype}, requires_grad={self.requires_grad})"

    def __len__(self):
        return self.shape[0]

    # ---- in-place conversions: like the reference these mutate and return self
    # (mytorch/tensor.py:131-135, 2094-2104) ----
    def astype(self, dtype):
        self.data = self.data.astype(dtype)
        return self

    def to(self, device=None):
        return self

    def contiguous(self):
        return self

    def detach(self):
        return Tensor(self.data)

    # ---- ops ----
    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        src = self
        out = Tensor(self.data.reshape(*shape))
        if self.requires_grad and _grad_enabled:
            out.requires_grad = True
            out.grad_fn = lambda g: src._accumulate(g.reshape(src.shape))
            out.grad_fn_name = "<ReshapeBackward>"
            out._add_parents(src)
        return out

    view = reshape

    def __add__(self, other):
        if not isinstance(other, Tensor):
            raise TypeError("Tensor + scalar is not on the training path; use tensors")
        if other.shape != self.shape:
            raise ValueError(f"shapes must match for +: {self.shape} vs {other.shape}")
        a, b = self, other
        out_data = DeviceArray.empty(a.shape, a.dtype)
        _lib.add(a.data.ptr, b.data.ptr, out_data.ptr, a.data.size, a.data.code, stream())
        out = Tensor(out_data)
        if (a.requires_grad or b.requires_grad) and _grad_enabled:
            def _bw(g):
                # both sides receive the same gradient (mytorch/tensor.py:272-330);
                # a side that adopts the buffer forces a copy for the other
                owned = False
                if a.requires_grad:
                    owned = (not a.is_param) and a.grad is None
                    a._accumulate(g)
                if b.requires_grad:
                    b._accumulate(g.copy() if (owned and not b.is_param and b.grad is None) else g)
            out.requires_grad = True
            out.grad_fn = _bw
            out.grad_fn_name = "<AddBackward>"
            out._add_parents(a, b)
        return out

    def _scale(self, s):
        a = self
        out_data = a.data.copy()
        _lib.scale(out_data.ptr, float(s), out_data.size, out_data.code, stream())
        out = Tensor(out_data)
        if a.requires_grad and _grad_enabled:
            def _bw(g):
                gs = g.copy()
                _lib.scale(gs.ptr, float(s), gs.size, gs.code, stream())
                a._accumulate(gs)
            out.requires_grad = True
            out.grad_fn = _bw
            out.grad_fn_name = "<MulBackward>"
            out._add_parents(a)
        return out

    def __mul__(self, s):
        if isinstance(s, Tensor):
            raise TypeError("elementwise Tensor*Tensor is not on the training path")
        return self._scale(s)

    __rmul__ = __mul__

    def __truediv__(self, s):
        return self._scale(1.0 / float(s))


def _factory(fill):
    def make(shape, requires_grad=False, dtype="float32", device=None):
        if isinstance(shape, int):
            shape = (shape,)
        arr = DeviceArray.zeros(shape, dtype) if fill == 0 else DeviceArray.empty(shape, dtype).fill_(fill)
        return Tensor(arr, requires_grad=requires_grad)
    return make


zeros = _factory(0)
ones = _factory(1)


def zeros_like(t, requires_grad=False):
    return Tensor(DeviceArray.zeros(t.shape, t.dtype), requires_grad=requires_grad)


def randn(shape, requires_grad=False, dtype="float32"):
    """Normal samples drawn on the host with NumPy's global generator, as the
    reference does (mytorch/_array.py:566-597), so seeds stay transferable."""
    return Tensor(DeviceArray.from_numpy(np.random.randn(*shape).astype(np.float32), dtype), requires_grad=requires_grad)


def arange(start, end=None, dtype="int32"):
    if end is None:
        start, end = 0, start
    return Tensor(DeviceArray.from_numpy(np.arange(start, end), dtype))
