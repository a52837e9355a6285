"""NCCL communicator for one-process-per-GPU data parallelism: the
`cupyx.distributed.NCCLBackend` surface the reference uses
(mytorch/accelerate.py:154-159 init, :249-250 broadcast, :732-772 all_reduce,
:873-880 barrier, :1050-1052 stop), on top of mt_comm_* of the C ABI.

Rendezvous is a one-shot TCP exchange on host:port (the role of cupyx's TCP
store): rank 0 creates the 128-byte NCCL id, serves it to the other ranks and
every rank then joins the communicator. The exchange has deadlines on every
socket operation, so a rank that never shows up produces an error, not a hang.

Gradient all-reduce runs on a dedicated non-blocking stream and overlaps the
backward pass of the last micro-batch: autograd reports each parameter as soon
as the last kernel writing its gradient has been queued; when all parameters of
a bucket of the flat gradient buffer have reported, the compute stream records
an event, the comm stream waits for it and reduces that bucket in place
(average). The compute stream waits for the comm stream before the first
kernel that reads gradients (norm / inf scan / AdamW).
"""
import ctypes as C
import socket
import struct
import time

from .. import _lib
from ..array import DeviceArray, stream

_OPS = {"sum": 0, "max": 1, "avg": 2}


def plan_buckets(total_elems, bucket_elems):
    """Splits [0, total) into contiguous (offset, count) buckets of at most
    bucket_elems elements (the last one may be smaller)."""
    if total_elems <= 0:
        return []
    bucket_elems = max(1, int(bucket_elems))
    return [(o, min(bucket_elems, total_elems - o)) for o in range(0, total_elems, bucket_elems)]


def exchange_unique_id(rank, world_size, host, port, make_id, timeout=120.0):
    """Rank 0 calls make_id() -> 128 bytes and serves it to world_size-1 peers;
    other ranks connect (retrying until `timeout`) and read it. Each peer sends
    its rank first so a stray connection is rejected."""
    if world_size == 1:
        return make_id()
    deadline = time.time() + timeout
    if rank == 0:
        uid = make_id()
        assert len(uid) == 128
        srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.bind((host, port))
        srv.listen(world_size)
        served = set()
        try:
            while len(served) < world_size - 1:
                remaining = deadline - time.time()
                if remaining <= 0:
                    raise TimeoutError(f"rendezvous: only {len(served) + 1} of {world_size} ranks arrived within {timeout}s")
                srv.settimeout(remaining)
                try:
                    conn, _ = srv.accept()
                except socket.timeout:
                    continue
                with conn:
                    conn.settimeout(10.0)
                    try:
                        hdr = conn.recv(8, socket.MSG_WAITALL)
                        magic, peer = struct.unpack("<II", hdr)
                        if magic != 0x4D54424E or not (0 < peer < world_size) or peer in served:
                            continue
                        conn.sendall(uid)
                        served.add(peer)
                    except (socket.timeout, struct.error, OSError):
                        continue
        finally:
            srv.close()
        return uid
    last = None
    while time.time() < deadline:
        try:
            with socket.create_connection((host, port), timeout=5.0) as s:
                s.settimeout(10.0)
                s.sendall(struct.pack("<II", 0x4D54424E, rank))
                buf = b""
                while len(buf) < 128:
                    chunk = s.recv(128 - len(buf))
                    if not chunk:
                        raise ConnectionError("rank 0 closed the connection early")
                    buf += chunk
                return buf
        except (ConnectionError, OSError, socket.timeout) as e:
            last = e
            time.sleep(0.2)
    raise TimeoutError(f"rendezvous: rank {rank} could not reach rank 0 at {host}:{port} within {timeout}s ({last})")


class NCCLBackend:
    def __init__(self, n_devices, rank, host="127.0.0.1", port=13333, timeout=120.0):
        self.world_size, self.rank = n_devices, rank

        def make_id():
            buf = C.create_string_buffer(128)
            _lib.comm_unique_id(buf)
            return buf.raw
        uid = exchange_unique_id(rank, n_devices, host, int(port), make_id, timeout)
        h = C.c_void_p()
        _lib.comm_init(C.byref(h), uid, rank, n_devices)
        self.handle = h
        s = C.c_void_p()
        _lib.stream_create(C.byref(s))
        self.comm_stream = s
        self._ev_ready = self._new_event()
        self._ev_done = self._new_event()
        self._bucket_events = []
        self._ov_active = False
        # With record_exposed set, every gradient sync leaves a pair of events: the compute stream's
        # position when it starts waiting, and the end of the last reduction on the comm stream.
        # exposed_ms() turns the pairs into the time the compute stream actually waited.
        self.record_exposed = False
        self._exposed_pairs = []

    @staticmethod
    def _new_event():
        e = C.c_void_p()
        _lib.event_create(C.byref(e))
        return e

    # ---- collectives on the compute stream (small or one-off messages) ----
    def broadcast(self, arr, root=0):
        _lib.comm_broadcast(self.handle, arr.ptr, arr.size, arr.code, root, stream())

    def all_reduce(self, in_array, out_array, op="sum"):
        _lib.comm_allreduce(self.handle, in_array.ptr, out_array.ptr, in_array.size, in_array.code, _OPS[op], stream())

    def barrier(self):
        _lib.comm_barrier(self.handle, stream())

    def stop(self):
        if self.handle is not None:
            _lib.comm_destroy(self.handle)
            self.handle = None

    def abort(self):
        if self.handle is not None:
            _lib.comm_abort(self.handle)
            self.handle = None

    # ---- gradient sync on the side stream ----
    def begin_overlap(self, grad_flat, bucket_elems, param_ranges):
        """Arms per-bucket triggering for one backward pass. param_ranges maps
        id(param) -> (offset, count) in the flat gradient buffer. Each bucket is
        all-reduced (average, in place, on the comm stream) as soon as every
        parameter overlapping it has reported ready."""
        self._ov_flat = grad_flat
        self._ov_buckets = plan_buckets(grad_flat.size, bucket_elems)
        self._ov_pending = [0] * len(self._ov_buckets)
        self._ov_launched = [False] * len(self._ov_buckets)
        self._ov_param_buckets = {}
        for pid, (off, cnt) in param_ranges.items():
            first = off // max(1, bucket_elems)
            last = (off + max(cnt, 1) - 1) // max(1, bucket_elems)
            bl = list(range(first, min(last, len(self._ov_buckets) - 1) + 1))
            self._ov_param_buckets[pid] = bl
            for b in bl:
                self._ov_pending[b] += 1
        while len(self._bucket_events) < len(self._ov_buckets):
            self._bucket_events.append(self._new_event())
        self._ov_active = True

    def param_ready(self, param):
        if not self._ov_active:
            return
        for b in self._ov_param_buckets.pop(id(param), ()):
            self._ov_pending[b] -= 1
            if self._ov_pending[b] == 0:
                self._launch_bucket(b)

    def _launch_bucket(self, b):
        if self._ov_launched[b]:
            return
        off, cnt = self._ov_buckets[b]
        ev = self._bucket_events[b]
        _lib.event_record(ev, stream())                    # gradients of this bucket are queued up to here
        _lib.stream_wait_event(self.comm_stream, ev)
        p = self._ov_flat.ptr + off * 4
        _lib.comm_allreduce(self.handle, p, p, cnt, _lib.F32, _OPS["avg"], self.comm_stream)
        self._ov_launched[b] = True

    def finish_overlap(self):
        """Launches whatever has not been triggered and makes the compute stream
        wait for all bucket reductions."""
        for b in range(len(self._ov_buckets)):
            self._launch_bucket(b)
        self._join_compute_stream()
        self._ov_active = False

    def _join_compute_stream(self):
        done = self._ev_done
        if self.record_exposed:
            arrived, done = self._new_event(), self._new_event()
            _lib.event_record(arrived, stream())
            self._exposed_pairs.append((arrived, done))
        _lib.event_record(done, self.comm_stream)
        _lib.stream_wait_event(stream(), done)

    def exposed_ms(self):
        """Mean over the recorded gradient syncs of max(0, end of the last reduction - moment the
        compute stream began to wait), in ms; clears the records. Call with the device idle."""
        waits = []
        for arrived, done in self._exposed_pairs:
            _lib.event_sync(done)
            ms = C.c_float()
            _lib.event_elapsed_ms(arrived, done, C.byref(ms))
            waits.append(max(0.0, ms.value))
            _lib.event_destroy(arrived)
            _lib.event_destroy(done)
        self._exposed_pairs = []
        return sum(waits) / len(waits) if waits else 0.0

    def allreduce_grads(self, grad_flat, bucket_elems):
        """In-place mean of the flat fp32 gradient buffer across ranks, bucket by
        bucket on the comm stream, then the compute stream waits for it."""
        _lib.event_record(self._ev_ready, stream())
        _lib.stream_wait_event(self.comm_stream, self._ev_ready)
        for off, cnt in plan_buckets(grad_flat.size, bucket_elems):
            p = grad_flat.ptr + off * 4
            _lib.comm_allreduce(self.handle, p, p, cnt, _lib.F32, _OPS["avg"], self.comm_stream)
        self._join_compute_stream()
