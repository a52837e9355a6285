"""ctypes binding of libmytorch_b200.so (the C ABI in include/mytorch_b200.h).

The library is the product: nothing here computes. If the shared object is
missing the import fails with instructions to build it; there is no fallback.
Every `mt_*` function that returns a status is wrapped so that a non-zero code
raises `MTError` carrying `mt_last_error()`.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmytorch_b200.so")

F32, F16, BF16 = 0, 1, 2
ACT = {None: 0, "none": 0, "gelu": 1, "relu_squared": 2, "relu2": 2, "relu": 3}
# aux_mode of mt_gemm_ex that multiplies by the derivative of an activation
ACT_BWD_AUX = {"gelu": 2, "relu_squared": 3, "relu2": 3, "relu": 4}


class MTError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"mytorch_b200 error {code}: {text}")
        self.code = code


class Strides3(C.Structure):
    _fields_ = [("b", C.c_int64), ("h", C.c_int64), ("s", C.c_int64)]


class TensorList(C.Structure):
    _fields_ = [("p", C.c_void_p), ("g", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
                ("p_half", C.c_void_p), ("size", C.c_void_p), ("weight_decay", C.c_void_p),
                ("chunk_tensor", C.c_void_p), ("chunk_offset", C.c_void_p),
                ("n_tensors", C.c_int64), ("n_chunks", C.c_int64)]


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python mytorch_b200/csrc/build.py` "
        "(nvcc, sm_100a). mytorch_b200 has no CPU or PyTorch fallback.")

lib = C.CDLL(LIB_PATH)

_p, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t
_pp = C.POINTER(C.c_void_p)
_S = Strides3

# name -> argtypes (all return int status unless listed in _RAW)
_SIG = {
    "mt_device_count": [C.POINTER(_i)],
    "mt_set_device": [_i],
    "mt_get_device": [C.POINTER(_i)],
    "mt_device_sm_count": [C.POINTER(_i)],
    "mt_malloc": [_pp, _sz, _p],
    "mt_free": [_p, _p],
    "mt_host_alloc": [_pp, _sz],
    "mt_host_free": [_p],
    "mt_memcpy_h2d": [_p, _p, _sz, _p],
    "mt_memcpy_d2h": [_p, _p, _sz, _p],
    "mt_memcpy_d2d": [_p, _p, _sz, _p],
    "mt_memset": [_p, _i, _sz, _p],
    "mt_stream_create": [_pp],
    "mt_stream_destroy": [_p],
    "mt_stream_sync": [_p],
    "mt_device_sync": [],
    "mt_event_create": [_pp],
    "mt_event_destroy": [_p],
    "mt_event_record": [_p, _p],
    "mt_event_sync": [_p],
    "mt_event_elapsed_ms": [_p, _p, C.POINTER(_f)],
    "mt_stream_wait_event": [_p, _p],
    "mt_mem_info": [C.POINTER(_sz), C.POINTER(_sz)],
    "mt_device_flag_read": [C.POINTER(_i), _p],
    "mt_range_push": [C.c_char_p],
    "mt_range_pop": [],
    "mt_prof_begin": [_i],
    "mt_prof_end": [C.POINTER(C.c_double), C.POINTER(_i64), C.POINTER(C.c_double)],
    "mt_cast": [_p, _i, _p, _i, _i64, _p],
    "mt_widen_u16_i32": [_p, _p, _i64, _p],
    "mt_softcap": [_p, _p, _i64, _f, _i, _p],
    "mt_fill": [_p, _i, _f, _i64, _p],
    "mt_add": [_p, _p, _p, _i64, _i, _p],
    "mt_axpby": [_p, _f, _p, _f, _i64, _i, _i, _p],
    "mt_scale": [_p, _f, _i64, _i, _p],
    "mt_add_rowvec": [_p, _p, _p, _i64, _i64, _i, _p],
    "mt_colsum": [_p, _p, _i64, _i64, _i, _i, _i, _p],
    "mt_sum_f32": [_p, _i, _i64, _p, _p],
    "mt_copy_strided": [_p, _p, _i, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64), _i, _i, _p],
    "mt_mul": [_p, _p, _p, _i64, _i, _p],
    "mt_rowsum": [_p, _p, _i64, _i64, _f, _i, _p],
    "mt_act_fwd": [_p, _p, _i64, _i, _i, _p],
    "mt_act_bwd": [_p, _p, _p, _i64, _i, _i, _p],
    "mt_layernorm_fwd": [_p, _p, _p, _p, _p, _p, _i64, _i64, _f, _i, _p],
    "mt_layernorm_bwd": [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i, _i, _p],
    "mt_layernorm_bwd_noalloc": [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i, _i, _p],
    "mt_rmsnorm_fwd": [_p, _p, _p, _p, _i64, _i64, _f, _i, _p],
    "mt_rmsnorm_bwd": [_p, _p, _p, _p, _p, _p, _i64, _i64, _i, _i, _p],
    "mt_softmax_fwd": [_p, _p, _i64, _i64, _i, _p],
    "mt_softmax_bwd": [_p, _p, _p, _i64, _i64, _i, _p],
    "mt_ce_fwd": [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _f, _i, _p],
    "mt_ce_bwd": [_p, _p, _p, _p, _f, _p, _p, _i64, _i64, _i64, _f, _i, _p],
    "mt_ce_fwd_grad": [_p, _p, _p, _p, _p, _p, _p, _f, _p, _i64, _i64, _i64, _f, _i, _p],
    "mt_scale_ratio": [_p, _i64, _p, _p, _i, _p],
    "mt_ce_chunk_fwd": [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _p],
    "mt_ce_chunk_finish": [_p, _p, _p, _p, _p, _p, _p, _i64, _p],
    "mt_ce_chunk_bwd": [_p, _p, _p, _p, _f, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _p],
    "mt_embedding_fwd": [_p, _p, _p, _i64, _i64, _i64, _i, _p],
    "mt_embedding_bwd": [_p, _p, _p, _p, _i64, _i64, _i64, _i, _p],
    "mt_embedding_pos_fwd": [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i, _p],
    "mt_pos_embedding_bwd": [_p, _p, _i64, _i64, _i64, _i, _p],
    "mt_rope": [_p, _p, _p, _i64, _i64, _i64, _i64, _i, _i, _p],
    "mt_rope_rmsnorm_fwd": [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _f, _i, _p],
    "mt_rope_rmsnorm_bwd": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i, _p],
    "mt_gemm": [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _i, _f, _i, _p],
    "mt_gemm_ex": [_p, _p, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _i, _f, _i, _p],
    "mt_gemm_force_simt": [_i],
    "mt_gemm_tile_policy": [_i],
    "mt_attn_fwd": [_p, _p, _p, _p, _p, _S, _S, _S, _S, _i64, _i64, _i64, _i64, _f, _i, _i, _p],
    "mt_attn_bwd": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _S, _S, _S, _S, _S, _S, _S, _S,
                    _i64, _i64, _i64, _i64, _f, _i, _i, _p],
    "mt_attn_fwd_gqa": [_p, _p, _p, _p, _p, _S, _S, _S, _S, _i64, _i64, _i64, _i64, _i64, _f, _i, _i, _p],
    "mt_attn_bwd_gqa": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _S, _S, _S, _S, _S, _S, _S, _S,
                        _i64, _i64, _i64, _i64, _i64, _f, _i, _i, _p],
    "mt_attn_force_simt": [_i],
    "mt_attn_decode": [_p, _p, _p, _p, _S, _S, _S, _i64, _i64, _i64, _i64, _i64, _f, _i, _i, _p],
    "mt_attn_decode_gqa": [_p, _p, _p, _p, _S, _S, _S, _i64, _i64, _i64, _i64, _i64, _i64, _f, _i, _i, _p],
    "mt_kv_append": [_p, _p, _p, _p, _S, _S, _S, _i64, _i64, _i64, _i64, _i64, _i64, _i, _p],
    "mt_gradnorm_multi": [C.POINTER(TensorList), _i, _p, _p, _p, _p],
    "mt_adamw_multi": [C.POINTER(TensorList), _i, _i, _f, C.c_double, C.c_double, _f, _p, _p, _f, _p, _i, _p, _i, _p],
    "mt_scaler_update": [_p, _p, _f, _f, _i, _f, _i, _p],
    "mt_comm_unique_id": [_p],
    "mt_comm_init": [_pp, _p, _i, _i],
    "mt_comm_broadcast": [_p, _p, _i64, _i, _i, _p],
    "mt_comm_allreduce": [_p, _p, _p, _i64, _i, _i, _p],
    "mt_comm_barrier": [_p, _p],
    "mt_comm_abort": [_p],
    "mt_comm_destroy": [_p],
}
# functions that do not return a status code
_RAW = {
    "mt_last_error": ([], C.c_char_p),
    "mt_version": ([], _i),
    "mt_launch_count": ([], _i64),
    "mt_embedding_bwd_scratch_bytes": ([_i64], _sz),
}

lib.mt_last_error.restype = C.c_char_p


def _checked(name, fn):
    def call(*args):
        rc = fn(*args)
        if rc != 0:
            raise MTError(rc, (lib.mt_last_error() or b"").decode(errors="replace") + f" [{name}]")
    call.__name__ = name
    return call


_g = globals()
for _name, _args in _SIG.items():
    _fn = getattr(lib, _name)
    _fn.argtypes = _args
    _fn.restype = _i
    _g[_name[3:]] = _checked(_name, _fn)
for _name, (_args, _res) in _RAW.items():
    _fn = getattr(lib, _name)
    _fn.argtypes = _args
    _fn.restype = _res
    _g[_name[3:]] = _fn

DECLARED = sorted(list(_SIG) + list(_RAW))


# ---- optional tracing of every compute call (environment variable MT_TRACE) ---------------------
# MT_TRACE=nvtx  one NVTX range per library call, named after the function (timeline profilers)
# MT_TRACE=time  a pair of CUDA events on the compute stream around every call; trace_report()
#                (also run at interpreter exit) prints calls and device milliseconds per function.
# Unset (the default) nothing is wrapped: the bindings above are used as they are.
# Runtime plumbing (allocation, copies, streams, events, communicator set-up) is never wrapped.
_TRACE = os.environ.get("MT_TRACE", "").strip().lower()
_NOT_TRACED = {"mt_device_count", "mt_set_device", "mt_get_device", "mt_device_sm_count", "mt_malloc", "mt_free",
               "mt_host_alloc", "mt_host_free", "mt_memcpy_h2d", "mt_memcpy_d2h", "mt_memcpy_d2d", "mt_stream_create",
               "mt_stream_destroy", "mt_stream_sync", "mt_device_sync", "mt_event_create", "mt_event_destroy",
               "mt_event_record", "mt_event_sync", "mt_event_elapsed_ms", "mt_stream_wait_event", "mt_mem_info",
               "mt_device_flag_read", "mt_range_push", "mt_range_pop", "mt_prof_begin", "mt_prof_end",
               "mt_gemm_force_simt", "mt_gemm_tile_policy", "mt_attn_force_simt", "mt_comm_unique_id",
               "mt_comm_init", "mt_comm_abort", "mt_comm_destroy"}
TRACED = sorted(n for n in _SIG if n not in _NOT_TRACED)


class _OpTimer:
    """Device time per library function: events are recorded on the compute stream around each
    call and read back in batches (one synchronisation per batch, none per call)."""
    BATCH = 4096

    def __init__(self):
        self.pending, self.spare, self.table = [], [], {}

    def _event(self):
        if self.spare:
            return self.spare.pop()
        e = C.c_void_p()
        _g["event_create"](C.byref(e))
        return e

    def wrap(self, name, fn):
        def call(*args):
            from .array import stream
            e0, e1 = self._event(), self._event()
            _g["event_record"](e0, stream())
            try:
                return fn(*args)
            finally:
                _g["event_record"](e1, stream())
                self.pending.append((name, e0, e1))
                if len(self.pending) >= self.BATCH:
                    self.collect()
        call.__name__ = name
        return call

    def collect(self):
        ms = C.c_float()
        for name, e0, e1 in self.pending:
            _g["event_sync"](e1)
            _g["event_elapsed_ms"](e0, e1, C.byref(ms))
            row = self.table.setdefault(name, [0.0, 0])
            row[0] += ms.value
            row[1] += 1
            self.spare += [e0, e1]
        self.pending = []

    def report(self, top=25, file=None):
        import sys
        self.collect()
        rows = sorted(((v[0], v[1], k) for k, v in self.table.items()), reverse=True)
        out = file or sys.stderr
        total = sum(r[0] for r in rows) or 1.0
        for ms, calls, name in rows[:top if top > 0 else None]:
            print(f"{name:28s} calls={calls:7d} total={ms:10.3f} ms avg={1e3 * ms / calls:9.1f} us share={100 * ms / total:5.1f}%", file=out)
        return [(name, calls, ms) for ms, calls, name in rows]


def _nvtx_wrap(name, fn):
    label = name.encode()

    def call(*args):
        lib.mt_range_push(label)
        try:
            return fn(*args)
        finally:
            lib.mt_range_pop()
    call.__name__ = name
    return call


_timer = None
if _TRACE == "nvtx":
    for _name in TRACED:
        _g[_name[3:]] = _nvtx_wrap(_name, _g[_name[3:]])
elif _TRACE == "time":
    import atexit
    _timer = _OpTimer()
    for _name in TRACED:
        _g[_name[3:]] = _timer.wrap(_name, _g[_name[3:]])
    atexit.register(lambda: _timer.report() if _timer.table or _timer.pending else None)
elif _TRACE:
    raise ImportError(f"MT_TRACE={_TRACE!r}: expected 'nvtx' or 'time'")


def trace_report(top=25, file=None):
    """With MT_TRACE=time: prints and returns [(function, calls, device milliseconds)], largest
    first, for the calls made so far. Raises when the timer is not on."""
    if _timer is None:
        raise RuntimeError("the per-call timer is off: set MT_TRACE=time before importing mytorch_b200")
    return _timer.report(top, file)


def device_count():
    n = C.c_int(0)
    lib.mt_device_count(C.byref(n))
    return n.value


def require_device():
    if device_count() == 0:
        raise MTError(3, "no CUDA device: mytorch_b200 runs on B200 (sm_100a) only, there is no CPU path")
