"""Reverse-mode autograd over device arrays: the `Tensor` of the reference
(mytorch/tensor.py:26-261) thinned to what the GPT training step uses.

The fused path of the GPT models goes through `mytorch_b200.nn.functional`; the methods below
are the general-purpose glue the reference's model files also use (transpose, chunk, matmul,
slicing, elementwise arithmetic, sums), so that e.g. the non-fused attention branch of
gpt2_trainer/gpt2.py:168-203 runs unchanged. Arrays are always contiguous: ops that the
reference expresses as views plus `.contiguous()` copy once, through one strided-copy kernel.

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


def _contig_strides(shape):
    st, acc = [], 1
    for n in reversed(shape):
        st.append(acc)
        acc *= n
    return tuple(reversed(st))


def _strided_copy(src, dst, shape, src_strides, dst_strides, src_offset=0, dst_offset=0, accumulate=False):
    """dst[dst_offset + idx.dst_strides] (+)= src[src_offset + idx.src_strides] over `shape`
    (element offsets and strides); one kernel (mt_copy_strided)."""
    import ctypes as C
    shape = [int(n) for n in shape] or [1]
    ss = [int(v) for v in src_strides] or [0]
    ds = [int(v) for v in dst_strides] or [0]
    # merge trailing dimensions that are contiguous on both sides; keeps most copies within 6 dims
    while len(shape) > 1 and ss[-2] == ss[-1] * shape[-1] and ds[-2] == ds[-1] * shape[-1]:
        n = shape.pop()
        s_, d_ = ss.pop(), ds.pop()
        shape[-1] *= n
        ss[-1], ds[-1] = s_, d_
    nd = len(shape)
    arr = C.c_int64 * nd
    item = src.itemsize
    _lib.copy_strided(src.ptr + src_offset * item, dst.ptr + dst_offset * item, nd, arr(*shape), arr(*ss), arr(*ds),
                      item, dst.code if accumulate else -1, stream())


def _norm_dim(d, ndim):
    d = int(d)
    if not -ndim <= d < ndim:
        raise IndexError(f"dimension {d} out of range for a {ndim}-d tensor")
    return d % ndim


def _graph(out, parents, fn, name):
    out.requires_grad = True
    out.grad_fn, out.grad_fn_name = fn, name
    out._add_parents(*parents)
    return out


def _wants_graph(*ts):
    return _grad_enabled and any(isinstance(t, Tensor) and t.requires_grad for t in ts)


class Tensor:
    # Optional callable(param) invoked during backward() as soon as the last closure contributing to
    # a parameter's gradient has run (set by Accelerator to start that gradient's all-reduce early).
    param_ready_hook = None
    # Device scalar that loss.backward() will be called with (the loss scale of mixed-precision
    # training), announced by the Accelerator so that a loss may fold it into a gradient it
    # produces already in its forward pass. None = backward() is expected with its default of 1.
    loss_grad_hint = None
    _unit_grad_ptr = None
    last_backward_timings = None

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

    def backward(self, grad=None, retain_graph=False, time_backward=False, num_ops_to_show=-1):
        """Topological sort from this tensor, closures run in reverse order;
        the graph is released afterwards (mytorch/tensor.py:182-261).

        time_backward=True brackets every closure with a pair of CUDA events on the compute stream
        and prints, after one synchronisation at the end, the device time per `grad_fn_name`
        (summed over its occurrences) - the reference's per-closure timer (:221-261), which
        synchronises after every closure and keeps only the last occurrence's time. The table is
        also left in `Tensor.last_backward_timings` ({name: [milliseconds, calls]})."""
        if retain_graph:
            raise NotImplementedError("retain_graph is not built: closures release their buffers as they run")
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
        marks = [] if time_backward else None
        for k, node in enumerate(exec_order):
            if node.grad_fn is not None:
                if marks is not None:
                    import ctypes as C
                    e0, e1 = C.c_void_p(), C.c_void_p()
                    _lib.event_create(C.byref(e0)); _lib.event_create(C.byref(e1))
                    _lib.event_record(e0, stream())
                node.grad_fn(node.grad)
                if marks is not None:
                    _lib.event_record(e1, stream())
                    marks.append((node.grad_fn_name or "<unnamed>", e0, e1))
                node.grad_fn = None
                node._parents = ()
                if not node.is_param:
                    node.grad = None      # activations' gradients are consumed
            if hook is not None:
                for p in ready_at.get(k, ()):
                    hook(p)               # every kernel writing p.grad has been queued
        if marks is not None:
            import ctypes as C
            table = {}
            for name, e0, e1 in marks:
                _lib.event_sync(e1)
                ms = C.c_float()
                _lib.event_elapsed_ms(e0, e1, C.byref(ms))
                row = table.setdefault(name, [0.0, 0])
                row[0] += ms.value
                row[1] += 1
                _lib.event_destroy(e0); _lib.event_destroy(e1)
            Tensor.last_backward_timings = table
            rows = sorted(table.items(), key=lambda kv: -kv[1][0])
            if num_ops_to_show is not None and num_ops_to_show >= 0:
                rows = rows[:num_ops_to_show]
            print(f"\nTop {num_ops_to_show} most time-consuming backward functions:")
            for name, (ms, n) in rows:
                print(f"{name:<34s} {ms:9.3f} ms total over {n} call(s)")

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

    def _broadcast_to(self, shape):
        """A contiguous copy of this tensor's data expanded to `shape` (NumPy broadcasting rules)."""
        if tuple(shape) == self.shape:
            return self.data
        nd = len(shape)
        mine = (1,) * (nd - self.ndim) + self.shape
        st = (0,) * (nd - self.ndim) + _contig_strides(self.shape)
        for m, n in zip(mine, shape):
            if m != n and m != 1:
                raise ValueError(f"cannot broadcast {self.shape} to {tuple(shape)}")
        src_st = [0 if m == 1 and n != 1 else v for m, n, v in zip(mine, shape, st)]
        out = DeviceArray.empty(shape, self.dtype)
        _strided_copy(self.data, out, shape, src_st, _contig_strides(shape))
        return out

    def _reduce_to_shape(self, g):
        """Sums a gradient of a broadcast result back to this tensor's shape."""
        if g.shape == self.shape:
            return g
        mine = (1,) * (len(g.shape) - self.ndim) + self.shape
        j = 0
        while j < len(mine) and mine[j:] != g.shape[j:]:
            if mine[j] != 1:
                raise NotImplementedError("gradient of a broadcast over inner dimensions is not built; broadcast over "
                                          f"leading dimensions only ({self.shape} vs {g.shape})")
            j += 1
        rows = 1
        for n in g.shape[:j]:
            rows *= n
        out = DeviceArray.empty(self.shape or (1,), g.dtype)
        _lib.colsum(g.ptr, out.ptr, rows, max(1, self.data.size), g.code, out.code, 0, stream())
        return out.reshape(self.shape)

    def _binary(self, other, kernel, name, grad_a, grad_b):
        """out = kernel(a, b) elementwise with NumPy broadcasting; grad_x(g, a_data, b_data) -> dx."""
        if not isinstance(other, Tensor):
            raise TypeError(f"{name} needs two tensors")
        a, b = self, other
        if a.dtype != b.dtype:
            raise TypeError(f"{name}: dtypes differ ({a.dtype} vs {b.dtype}); cast one side with astype")
        shape = a.shape if a.shape == b.shape else tuple(np.broadcast_shapes(a.shape, b.shape))
        ad, bd = a._broadcast_to(shape), b._broadcast_to(shape)
        out_data = DeviceArray.empty(shape, a.dtype)
        kernel(ad, bd, out_data)
        out = Tensor(out_data)
        if _wants_graph(a, b):
            def _bw(g):
                if a.requires_grad:
                    a._accumulate(a._reduce_to_shape(grad_a(g, ad, bd)))
                if b.requires_grad:
                    b._accumulate(b._reduce_to_shape(grad_b(g, ad, bd)))
            _graph(out, (a, b), _bw, name)
        return out

    def __add__(self, other):
        if isinstance(other, (int, float)):
            raise TypeError("Tensor + scalar is not built; add tensors")
        add = lambda x, y, o: _lib.add(x.ptr, y.ptr, o.ptr, o.size, o.code, stream())
        # both sides receive the same gradient (mytorch/tensor.py:272-330); each gets its own buffer
        return self._binary(other, add, "<AddBackward>", lambda g, x, y: g, lambda g, x, y: g.copy())

    def __sub__(self, other):
        """mytorch/tensor.py:451."""
        def sub(x, y, o):
            o.copy_from(x)
            _lib.axpby(y.ptr, -1.0, o.ptr, 1.0, o.size, y.code, o.code, stream())

        def neg(g, x, y):
            n = g.copy()
            _lib.scale(n.ptr, -1.0, n.size, n.code, stream())
            return n
        return self._binary(other, sub, "<SubBackward>", lambda g, x, y: g, neg)

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
            _graph(out, (a,), _bw, "<MulBackward>")
        return out

    def __mul__(self, s):
        """Scalar multiple, or the elementwise product of two tensors (mytorch/tensor.py:596-640)."""
        if not isinstance(s, Tensor):
            return self._scale(s)

        def mul(x, y, o):
            _lib.mul(x.ptr, y.ptr, o.ptr, o.size, o.code, stream())

        def times(which):
            def f(g, x, y):
                o = DeviceArray.empty(g.shape, g.dtype)
                other = y if which == 0 else x
                _lib.mul(g.ptr, other.ptr, o.ptr, o.size, o.code, stream())
                return o
            return f
        return self._binary(s, mul, "<MulBackward>", times(0), times(1))

    __rmul__ = __mul__

    def __neg__(self):
        return self._scale(-1.0)

    def __truediv__(self, s):
        if isinstance(s, Tensor):
            raise TypeError("Tensor / Tensor is not built; divide by a scalar")
        return self._scale(1.0 / float(s))

    # ---- layout ----
    def transpose(self, dim1, dim2):
        """Swaps two dimensions (mytorch/tensor.py:1381); the result is a contiguous copy."""
        d1, d2 = _norm_dim(dim1, self.ndim), _norm_dim(dim2, self.ndim)
        if d1 == d2:
            return self
        perm = list(range(self.ndim))
        perm[d1], perm[d2] = perm[d2], perm[d1]
        return self.permute(*perm)

    def permute(self, *dims):
        if len(dims) == 1 and isinstance(dims[0], (tuple, list)):
            dims = tuple(dims[0])
        dims = [_norm_dim(d, self.ndim) for d in dims]
        if sorted(dims) != list(range(self.ndim)):
            raise ValueError(f"permute needs each dimension once, got {dims}")
        src = self
        st = _contig_strides(self.shape)
        shape = tuple(self.shape[d] for d in dims)
        out_data = DeviceArray.empty(shape, self.dtype)
        _strided_copy(self.data, out_data, shape, [st[d] for d in dims], _contig_strides(shape))
        out = Tensor(out_data)
        if _wants_graph(self):
            inv = [dims.index(i) for i in range(self.ndim)]

            def _bw(g):
                gst = _contig_strides(shape)
                back = DeviceArray.empty(src.shape, g.dtype)
                _strided_copy(g, back, src.shape, [gst[i] for i in inv], _contig_strides(src.shape))
                src._accumulate(back)
            _graph(out, (src,), _bw, "<PermuteBackward>")
        return out

    def _slices_node(self, pieces, name):
        """Outputs that are rectangular pieces of this tensor: `pieces` = [(offset, shape, strides)]
        in elements of this tensor's layout. One graph-only node collects the pieces' gradients and
        writes the parent's gradient once: pieces that cover it need no zero fill."""
        src = self
        outs = []
        for off, shp, st in pieces:
            o = DeviceArray.empty(shp, self.dtype)
            _strided_copy(self.data, o, shp, st, _contig_strides(shp), src_offset=off)
            outs.append(Tensor(o))
        if _wants_graph(self):
            slots = [None] * len(pieces)
            covered = sum(int(np.prod(shp)) for _, shp, _ in pieces) == self.data.size and len(pieces) > 1

            def _bw_join(_):
                full = all(s_ is not None for s_ in slots) and covered
                dt = next((s_.dtype for s_ in slots if s_ is not None), src.dtype)
                back = DeviceArray.empty(src.shape, dt) if full else DeviceArray.zeros(src.shape, dt)
                for (off, shp, st), g in zip(pieces, slots):
                    if g is not None:
                        _strided_copy(g, back, shp, _contig_strides(shp), st, dst_offset=off)     # pieces never overlap
                for i in range(len(slots)):
                    slots[i] = None
                src._accumulate(back)
            join = Tensor(self.data)
            _graph(join, (src,), _bw_join, name)

            def park(i):
                def f(g):
                    slots[i] = g
                return f
            for i, o in enumerate(outs):
                _graph(o, (join,), park(i), name)
        return outs

    def chunk(self, chunks, dim=0):
        """`chunks` equal pieces along `dim` (mytorch/tensor.py:1598-1660). The backward pass writes
        each piece's gradient into its place of one buffer (the reference pads every piece to the
        full size with zeros and adds the padded tensors)."""
        d = _norm_dim(dim, self.ndim)
        if self.shape[d] % chunks:
            raise ValueError(f"dimension {d} of size {self.shape[d]} does not split into {chunks} equal chunks")
        w = self.shape[d] // chunks
        st = _contig_strides(self.shape)
        shp = self.shape[:d] + (w,) + self.shape[d + 1:]
        return tuple(self._slices_node([(i * w * st[d], shp, st) for i in range(chunks)], "<ChunkBackward>"))

    def __getitem__(self, idx):
        """Basic indexing with integers, slices and `...` (mytorch/tensor.py:1314-1358): a copy of the
        selected block; the gradient is scattered back into zeros."""
        if not isinstance(idx, tuple):
            idx = (idx,)
        if any(i is Ellipsis for i in idx):
            k = idx.index(Ellipsis)
            idx = idx[:k] + (slice(None),) * (self.ndim - (len(idx) - 1)) + idx[k + 1:]
        idx = idx + (slice(None),) * (self.ndim - len(idx))
        if len(idx) != self.ndim:
            raise IndexError("too many indices")
        st = _contig_strides(self.shape)
        off, shp, sst = 0, [], []
        for i, n, s_ in zip(idx, self.shape, st):
            if isinstance(i, (int, np.integer)):
                i = int(i) + (n if i < 0 else 0)
                if not 0 <= i < n:
                    raise IndexError("index out of range")
                off += i * s_
            elif isinstance(i, slice):
                lo, hi, step = i.indices(n)
                cnt = max(0, (hi - lo + (step - (1 if step > 0 else -1))) // step)
                off += lo * s_
                shp.append(cnt)
                sst.append(s_ * step)
            else:
                raise TypeError("only integers, slices and ... are supported as indices")
        return self._slices_node([(off, tuple(shp), tuple(sst))], "<IndexBackward>")[0]

    # ---- reductions ----
    def sum(self, dim=None, keepdims=False):
        """Sum over all elements or over one dimension (mytorch/tensor.py:1734-1850)."""
        return self._reduce(dim, keepdims, mean=False)

    def mean(self, dim=None, keepdims=False):
        """mytorch/tensor.py:1852-1955."""
        return self._reduce(dim, keepdims, mean=True)

    def _reduce(self, dim, keepdims, mean):
        src = self
        if dim is None:
            flat, rows, cols = self.data, 1, self.data.size
            kd = (1,) * self.ndim
            out_shape = kd if keepdims else ()
        else:
            d = _norm_dim(dim, self.ndim)
            flat = self.data
            if d != self.ndim - 1:       # bring the reduced dimension last; the rows then come out in natural order
                perm = [i for i in range(self.ndim) if i != d] + [d]
                st = _contig_strides(self.shape)
                shp = tuple(self.shape[i] for i in perm)
                flat = DeviceArray.empty(shp, self.dtype)
                _strided_copy(self.data, flat, shp, [st[i] for i in perm], _contig_strides(shp))
            cols = self.shape[d]
            rows = self.data.size // max(1, cols)
            kd = self.shape[:d] + (1,) + self.shape[d + 1:]
            out_shape = kd if keepdims else self.shape[:d] + self.shape[d + 1:]
        alpha = 1.0 / max(1, cols) if mean else 1.0
        out_data = DeviceArray.empty((rows,), self.dtype)
        _lib.rowsum(flat.ptr, out_data.ptr, rows, cols, float(alpha), flat.code, stream())
        out = Tensor(out_data.reshape(out_shape))
        if _wants_graph(self):
            def _bw(g):
                back = Tensor(g.reshape(kd))._broadcast_to(src.shape)
                if back.ptr == g.ptr:
                    back = g.copy().reshape(src.shape)
                if alpha != 1.0:
                    _lib.scale(back.ptr, float(alpha), back.size, back.code, stream())
                src._accumulate(back)
            _graph(out, (src,), _bw, "<MeanBackward>" if mean else "<SumBackward>")
        return out

    # ---- matmul ----
    def __matmul__(self, other):
        """[..., M, K] @ [..., K, N] with equal leading dimensions, or a 2-d right operand shared by
        every batch (mytorch/tensor.py:735-774); each matrix product is one mt_gemm call."""
        from . import fused_ops as K
        a, b = self, other
        if not isinstance(b, Tensor) or a.ndim < 2 or b.ndim < 2:
            raise TypeError("@ needs two tensors of at least two dimensions")
        M, Kd = a.shape[-2:]
        Kb, N = b.shape[-2:]
        if Kd != Kb:
            raise ValueError(f"inner dimensions must match: {a.shape} @ {b.shape}")
        shared = b.ndim == 2
        if not shared and a.shape[:-2] != b.shape[:-2]:
            raise ValueError(f"leading dimensions must match: {a.shape} @ {b.shape}")
        batch = int(np.prod(a.shape[:-2])) if a.ndim > 2 else 1
        out_data = DeviceArray.empty(a.shape[:-2] + (M, N), a.dtype)

        def mats(arr, r, c, shared_=False):
            return [arr.flat_view(0 if shared_ else i * r * c, (r, c)) for i in range(batch)]
        if shared:
            K.gemm(a.data.reshape(batch * M, Kd), b.data, out=out_data.reshape(batch * M, N))
        else:
            for x, y, o in zip(mats(a.data, M, Kd), mats(b.data, Kd, N), mats(out_data, M, N)):
                K.gemm(x, y, out=o)
        out = Tensor(out_data)
        if _wants_graph(a, b):
            def _bw(g):
                if a.requires_grad:
                    da = DeviceArray.empty(a.shape, g.dtype)
                    if shared:
                        K.gemm(g.reshape(batch * M, N), b.data, trans_b=True, out=da.reshape(batch * M, Kd))
                    else:
                        for gi, y, o in zip(mats(g, M, N), mats(b.data, Kd, N), mats(da, M, Kd)):
                            K.gemm(gi, y, trans_b=True, out=o)                  # dA = dC B^T
                    a._accumulate(da)
                if b.requires_grad:
                    if shared:
                        db = K.gemm(a.data.reshape(batch * M, Kd), g.reshape(batch * M, N), trans_a=True,
                                    out_dtype="float32" if b.is_param else None)
                    else:
                        db = DeviceArray.empty(b.shape, g.dtype)
                        for x, gi, o in zip(mats(a.data, M, Kd), mats(g, M, N), mats(db, Kd, N)):
                            K.gemm(x, gi, trans_a=True, out=o)                  # dB = A^T dC
                    b._accumulate(db)
            _graph(out, (a, b), _bw, "<MatmulBackward>")
        return out


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
