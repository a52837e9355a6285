"""Device arrays for the C ABI: the CUDA backend of `Array`
(mytorch/_array.py:24-655 in the reference, where it is a cupy.ndarray).

A `DeviceArray` is a pointer + shape + dtype over memory from the library's
stream-ordered pool (`mt_malloc`), always C-contiguous. It exposes
`__cuda_array_interface__` (v3) so other CUDA libraries can read it in place,
and anything exposing that interface can be wrapped with `as_device_array`.
No arithmetic happens here: kernels are called through `mytorch_b200.fused_ops`
and `mytorch_b200.ops`.
"""
import ctypes as C
import math

import numpy as np

from . import _lib

_DT = {"float32": (_lib.F32, 4, np.float32), "float16": (_lib.F16, 2, np.float16),
       "bfloat16": (_lib.BF16, 2, np.uint16), "int32": (None, 4, np.int32),
       "int64": (None, 8, np.int64), "uint8": (None, 1, np.uint8)}
_TYPESTR = {"float32": "<f4", "float16": "<f2", "bfloat16": "<u2", "int32": "<i4", "int64": "<i8", "uint8": "|u1"}

_stream = None


def stream():
    """The process's compute stream (created on first use, non-blocking)."""
    global _stream
    if _stream is None:
        _lib.require_device()
        s = C.c_void_p()
        _lib.stream_create(C.byref(s))
        _stream = s
    return _stream


def set_stream(s):
    global _stream
    _stream = s


def synchronize():
    _lib.stream_sync(stream())


def norm_dtype(dt):
    if isinstance(dt, str):
        name = dt
    else:
        name = np.dtype(dt).name
    if name not in _DT:
        raise TypeError(f"unsupported dtype {dt!r}")
    return name


def code(dt):
    c = _DT[norm_dtype(dt)][0]
    if c is None:
        raise TypeError(f"{dt} is not a floating dtype of the library")
    return c


def f32_to_bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = u + 0x7FFF + ((u >> 16) & 1)
    return (rounded >> 16).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


class DeviceArray:
    __slots__ = ("ptr", "shape", "dtype", "_base", "_owns", "__weakref__")

    def __init__(self, ptr, shape, dtype, base=None, owns=False):
        self.ptr = int(ptr)
        self.shape = tuple(int(s) for s in shape)
        self.dtype = norm_dtype(dtype)
        self._base = base
        self._owns = owns

    # ---- construction ----
    @classmethod
    def empty(cls, shape, dtype="float32"):
        if isinstance(shape, int):
            shape = (shape,)
        dtype = norm_dtype(dtype)
        n = math.prod(shape) * _DT[dtype][1]
        p = C.c_void_p()
        _lib.malloc(C.byref(p), n, stream())
        return cls(p.value, shape, dtype, owns=True)

    @classmethod
    def zeros(cls, shape, dtype="float32"):
        a = cls.empty(shape, dtype)
        _lib.memset(a.ptr, 0, a.nbytes, stream())
        return a

    @classmethod
    def from_numpy(cls, a, dtype=None):
        """Host -> device. float64 becomes float32 and int64 becomes int32, the
        defaults of the reference Array (mytorch/_array.py:106-118)."""
        a = np.asarray(a)
        if dtype is None:
            if a.dtype == np.float64:
                dtype = "float32"
            elif a.dtype == np.int64:
                dtype = "int32"
            else:
                dtype = a.dtype.name
        dtype = norm_dtype(dtype)
        if dtype == "bfloat16":
            host = f32_to_bf16_bits(a)
        else:
            host = np.ascontiguousarray(a, dtype=_DT[dtype][2])
        out = cls.empty(a.shape, dtype)
        if host.nbytes:
            _lib.memcpy_h2d(out.ptr, host.ctypes.data, host.nbytes, stream())
            synchronize()  # `host` may be a temporary
        return out

    def __del__(self):
        if getattr(self, "_owns", False) and self.ptr and _stream is not None:
            try:
                _lib.lib.mt_free(C.c_void_p(self.ptr), _stream)
            except Exception:
                pass
            self._owns = False

    # ---- properties ----
    @property
    def size(self):
        return math.prod(self.shape)

    @property
    def itemsize(self):
        return _DT[self.dtype][1]

    @property
    def nbytes(self):
        return self.size * self.itemsize

    @property
    def ndim(self):
        return len(self.shape)

    @property
    def code(self):
        return code(self.dtype)

    @property
    def __cuda_array_interface__(self):
        return {"shape": self.shape, "typestr": _TYPESTR[self.dtype], "data": (self.ptr, False),
                "version": 3, "strides": None, "stream": int(stream().value or 0) or 1}

    # ---- views and copies ----
    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        if -1 in shape:
            known = -math.prod(shape)
            shape = tuple(self.size // known if s == -1 else s for s in shape)
        assert math.prod(shape) == self.size, (shape, self.shape)
        return DeviceArray(self.ptr, shape, self.dtype, base=self._base or self)

    def rows(self, start, stop):
        """View of rows [start, stop) along the first axis."""
        row_bytes = (self.size // self.shape[0]) * self.itemsize if self.shape[0] else 0
        return DeviceArray(self.ptr + start * row_bytes, (stop - start,) + self.shape[1:], self.dtype,
                           base=self._base or self)

    def flat_view(self, offset, shape, dtype=None):
        """View at an element offset of the flat buffer, with a new shape."""
        dtype = norm_dtype(dtype or self.dtype)
        return DeviceArray(self.ptr + offset * self.itemsize, shape, dtype, base=self._base or self)

    def numpy(self):
        host = np.empty(self.shape, dtype=_DT[self.dtype][2])
        if host.nbytes:
            _lib.memcpy_d2h(host.ctypes.data, self.ptr, host.nbytes, stream())
            synchronize()
        if self.dtype == "bfloat16":
            return bf16_bits_to_f32(host)
        return host

    def copy(self):
        out = DeviceArray.empty(self.shape, self.dtype)
        _lib.memcpy_d2d(out.ptr, self.ptr, self.nbytes, stream())
        return out

    def copy_from(self, other):
        assert other.nbytes == self.nbytes and other.dtype == self.dtype
        _lib.memcpy_d2d(self.ptr, other.ptr, self.nbytes, stream())
        return self

    def set_from_numpy(self, a):
        tmp = DeviceArray.from_numpy(np.asarray(a).reshape(self.shape), self.dtype)
        return self.copy_from(tmp)

    def astype(self, dtype):
        dtype = norm_dtype(dtype)
        if dtype == self.dtype:
            return self
        out = DeviceArray.empty(self.shape, dtype)
        _lib.cast(self.ptr, self.code, out.ptr, out.code, self.size, stream())
        return out

    def fill_(self, value):
        _lib.fill(self.ptr, self.code, float(value), self.size, stream())
        return self

    def zero_(self):
        _lib.memset(self.ptr, 0, self.nbytes, stream())
        return self

    def item(self):
        return self.numpy().reshape(-1)[0].item()

    def __repr__(self):
        return f"DeviceArray(shape={self.shape}, dtype={self.dtype}, ptr=0x{self.ptr:x})"


def as_device_array(x):
    """Wraps any object exposing `__cuda_array_interface__` (C-contiguous)."""
    if isinstance(x, DeviceArray):
        return x
    cai = x.__cuda_array_interface__
    if cai.get("strides") not in (None,):
        raise ValueError("only C-contiguous arrays can cross the C ABI")
    names = {v: k for k, v in _TYPESTR.items()}
    return DeviceArray(cai["data"][0], cai["shape"], names[cai["typestr"]], base=x)
