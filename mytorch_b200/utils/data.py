"""Input pipeline of the training step: Dataset, a threaded DataLoader and the token-window
dataset of the GPT-2 trainer, with the same interface as the reference
(mytorch/utils/data.py:12-345, gpt2_trainer/train_gpt2.py:145-170), plus device staging.

Differences from the reference, all on the side of determinism and overlap:
* batches are delivered in submission order whatever worker finishes first (the reference puts
  finished batches in a plain queue and notes that an ordered queue would be right);
* `TokenLoader` draws its windows from its own seeded generator (seed + rank), not from the
  global NumPy state shared with weight initialisation;
* with `device=True` a batch is copied to pinned host memory, sent host -> device on a copy stream
  while the previous step computes, and handed out as device Tensors that the compute stream
  waits for with an event; uint16 token ids cross PCIe as uint16 and are widened to int32 on the
  device (`mt_widen_u16_i32`). The device buffers belong to the loader and are reused: a batch
  stays valid until `staging_depth - 1` further batches have been requested.
"""
import ctypes as C
import threading

import numpy as np


class Dataset:
    """Anything with __len__ and __getitem__ (utils/data.py:12-18)."""

    def __len__(self):
        raise NotImplementedError

    def __getitem__(self, idx):
        raise NotImplementedError


def _to_host(x):
    if isinstance(x, np.ndarray):
        return x
    if hasattr(x, "numpy"):
        return np.asarray(x.numpy())
    return np.asarray(x)


class TokenLoader(Dataset):
    """Random windows of `context_length` tokens (and the same window shifted by one) from a flat
    uint16 token file (train_gpt2.py:145-170). `tokens` may be a path to a .bin file (memory
    mapped) or an array already in memory (synthetic data)."""

    def __init__(self, tokens, context_length, virtual_length=1 << 20, seed=0, rank=0):
        self.context_length = int(context_length)
        self.arr = np.memmap(tokens, dtype=np.uint16, mode="r") if isinstance(tokens, (str, bytes)) else np.asarray(tokens)
        self.num_tokens = int(self.arr.shape[0])
        if self.num_tokens < self.context_length + 2:
            raise ValueError("TokenLoader: fewer tokens than one window")
        self.virtual_length = int(virtual_length)
        self.seed, self.rank = int(seed), int(rank)

    def __len__(self):
        """Sampling is random, so the length only tells the loader how long an "epoch" is."""
        return self.virtual_length

    def __getitem__(self, idx):
        # the window depends only on (seed, rank, idx): any worker can produce any sample
        rng = np.random.default_rng((self.seed, self.rank, int(idx)))
        start = int(rng.integers(0, self.num_tokens - self.context_length - 1))
        x = self.arr[start:start + self.context_length]
        y = self.arr[start + 1:start + self.context_length + 1]
        return np.asarray(x), np.asarray(y)


class _Slot:
    """One staged batch: pinned host buffers, device buffers, the event of its copy."""
    __slots__ = ("pinned", "pinned_bytes", "dev", "event", "tensors", "busy")

    def __init__(self):
        self.pinned, self.pinned_bytes, self.dev, self.event, self.tensors, self.busy = [], [], [], None, None, None


class DataLoader:
    """Batches from `dataset`, optionally prepared by `num_workers` threads `prefetch_factor`
    batches ahead, collated by stacking along axis 0 (or `collate_fn`). Iteration, `len`,
    `state_dict` / `load_state_dict` (epoch, batches consumed, the epoch's index order) and
    `shutdown` behave as in utils/data.py:20-345. `device=True` adds the staged host -> device
    path described at the top of this file and yields `mytorch_b200.Tensor`s."""

    def __init__(self, dataset, batch_size=1, shuffle=False, num_workers=0, prefetch_factor=2, collate_fn=None,
                 timeout=30, device=False, staging_depth=2):
        self.dataset, self.batch_size, self.shuffle = dataset, int(batch_size), bool(shuffle)
        self.num_workers, self.prefetch = int(num_workers), int(prefetch_factor)
        self.collate_fn = collate_fn if collate_fn is not None else self.default_collate
        self.timeout = timeout
        self.indices = np.arange(len(dataset))
        self.lock = threading.Lock()
        self.cond = threading.Condition(self.lock)
        self.stop_signal = threading.Event()
        self.workers = []
        self.epoch, self.batches_consumed = 0, 0
        self._shuffled_indices, self._resume_from_state = None, False
        self._next_ticket, self._next_out, self._ready, self._n_batches = 0, 0, {}, 0
        self.device = bool(device)
        self._slots = [_Slot() for _ in range(max(2, int(staging_depth)))] if self.device else []
        self._staged = []           # slots in flight, oldest first
        self._copy_stream = None
        self._exhausted = False

    # ------------------------------------------------------------------ collate ----
    def default_collate(self, batch):
        if isinstance(batch[0], (tuple, list)):
            return tuple(self.default_collate([b[i] for b in batch]) for i in range(len(batch[0])))
        return np.stack([_to_host(b) for b in batch])

    def __len__(self):
        return (len(self.dataset) + self.batch_size - 1) // self.batch_size

    # ---------------------------------------------------------------- host side ----
    def _make_batch(self, ticket):
        lo = ticket * self.batch_size
        idx = [int(i) for i in self.indices[lo:lo + self.batch_size]]
        return self.collate_fn([self.dataset[i] for i in idx])

    def _worker_loop(self):
        while not self.stop_signal.is_set():
            with self.cond:
                # stay at most prefetch*workers batches ahead of the consumer
                while (not self.stop_signal.is_set() and self._next_ticket < self._n_batches and
                       self._next_ticket - self._next_out >= self.prefetch * self.num_workers):
                    self.cond.wait(0.05)
                if self.stop_signal.is_set() or self._next_ticket >= self._n_batches:
                    return
                ticket = self._next_ticket
                self._next_ticket += 1
            try:
                item = self._make_batch(ticket)
            except Exception as e:          # delivered to the consumer in order
                item = e
            with self.cond:
                self._ready[ticket] = item
                self.cond.notify_all()

    def __iter__(self):
        self.shutdown()
        self.stop_signal.clear()
        n = len(self.dataset)
        if self._resume_from_state:
            self.indices = self._shuffled_indices
            start = self.batches_consumed
            self._resume_from_state = False
        else:
            self.batches_consumed = 0
            self.indices = np.random.permutation(n) if self.shuffle else np.arange(n)
            self._shuffled_indices = self.indices.copy()
            start = 0
        self._n_batches = (n + self.batch_size - 1) // self.batch_size
        self._next_ticket = self._next_out = start
        self._ready, self._exhausted = {}, False
        self._staged = []
        for slot in self._slots:
            slot.tensors = None
        if self.num_workers > 0:
            self.workers = [threading.Thread(target=self._worker_loop, daemon=True) for _ in range(self.num_workers)]
            for t in self.workers:
                t.start()
        return self

    def _next_host_batch(self):
        """The next collated host batch in order, or None at the end of the epoch."""
        if self._next_out >= self._n_batches:
            return None
        ticket = self._next_out
        if self.num_workers == 0:
            item = self._make_batch(ticket)
        else:
            with self.cond:
                ok = self.cond.wait_for(lambda: ticket in self._ready, timeout=self.timeout)
                if not ok:
                    if not any(w.is_alive() for w in self.workers):
                        return None
                    raise RuntimeError(f"DataLoader timeout after {self.timeout}s. Workers may be blocked or dataset "
                                       f"loading is too slow. Try increasing timeout or reducing num_workers.")
                item = self._ready.pop(ticket)
        self._next_out += 1
        if self.num_workers > 0:
            with self.cond:
                self.cond.notify_all()
        if isinstance(item, Exception):
            raise item
        return item

    # -------------------------------------------------------------- device side ----
    def _stage(self, slot, batch):
        """pinned copy + asynchronous host -> device copy of one batch on the copy stream."""
        from .. import _lib
        from ..array import DeviceArray, synchronize
        from ..tensor import Tensor
        fields = list(batch) if isinstance(batch, (tuple, list)) else [batch]
        if self._copy_stream is None:
            s = C.c_void_p()
            _lib.stream_create(C.byref(s))
            self._copy_stream = s
        if slot.event is None:
            e = C.c_void_p()
            _lib.event_create(C.byref(e))
            slot.event = e
        if slot.busy is not None:       # the consumer's kernels on the previous occupant have been enqueued
            _lib.stream_wait_event(self._copy_stream, slot.busy)
        while len(slot.pinned) < len(fields):
            slot.pinned.append(None); slot.pinned_bytes.append(0); slot.dev.append(None)
        tensors = []
        for k, a in enumerate(fields):
            a = np.ascontiguousarray(_to_host(a))
            if a.dtype == np.int64:
                a = a.astype(np.int32)
            elif a.dtype == np.float64:
                a = a.astype(np.float32)
            if slot.pinned_bytes[k] < a.nbytes:
                if slot.pinned[k] is not None:
                    _lib.stream_sync(self._copy_stream)
                    _lib.host_free(slot.pinned[k])
                p = C.c_void_p()
                _lib.host_alloc(C.byref(p), max(a.nbytes, 16))
                slot.pinned[k], slot.pinned_bytes[k] = p, a.nbytes
            C.memmove(slot.pinned[k], a.ctypes.data, a.nbytes)
            widen = a.dtype == np.uint16
            key = (a.shape, a.dtype.name)
            if slot.dev[k] is None or slot.dev[k][0] != key:
                # device buffers are owned by the slot and reused; they come from the compute
                # stream's pool, so the copy stream may only touch them once that stream has
                # passed the allocation
                raw = DeviceArray.empty((a.nbytes,), "uint8") if widen else DeviceArray.empty(a.shape, a.dtype.name)
                out = DeviceArray.empty(a.shape, "int32") if widen else raw
                synchronize()
                slot.dev[k] = (key, raw, out)
            _, raw, out = slot.dev[k]
            _lib.memcpy_h2d(raw.ptr, slot.pinned[k], a.nbytes, self._copy_stream)
            if widen:
                _lib.widen_u16_i32(raw.ptr, out.ptr, a.size, self._copy_stream)
            tensors.append(Tensor(out))
        _lib.event_record(slot.event, self._copy_stream)
        slot.tensors = tuple(tensors) if isinstance(batch, (tuple, list)) else tensors[0]

    def _next_device_batch(self):
        from .. import _lib
        from ..array import stream
        # the batch handed out last time: everything that reads it is on the compute stream by now
        if self._staged and self._staged[0].tensors is None:
            done = self._staged.pop(0)
            if done.busy is None:
                e = C.c_void_p()
                _lib.event_create(C.byref(e))
                done.busy = e
            _lib.event_record(done.busy, stream())
        free = [s for s in self._slots if s not in self._staged]
        while free and not self._exhausted:
            batch = self._next_host_batch()
            if batch is None:
                self._exhausted = True
                break
            slot = free.pop(0)
            self._stage(slot, batch)
            self._staged.append(slot)
        if not self._staged:
            return None
        slot = self._staged[0]
        _lib.stream_wait_event(stream(), slot.event)
        out, slot.tensors = slot.tensors, None
        return out

    def __next__(self):
        batch = self._next_device_batch() if self.device else self._next_host_batch()
        if batch is None:
            self.reset_epoch()
            self.shutdown()
            raise StopIteration
        self.batches_consumed += 1
        return batch

    # ------------------------------------------------------------- bookkeeping ----
    def shutdown(self):
        self.stop_signal.set()
        with self.cond:
            self.cond.notify_all()
        for t in self.workers:
            t.join(timeout=5)
        self.workers = []
        self._ready = {}

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass

    def reset_epoch(self):
        if self.batches_consumed != 0 and self._shuffled_indices is not None:
            self.epoch += 1
            self.batches_consumed = 0
            self._shuffled_indices = None

    def state_dict(self):
        """Where the loader stands, to resume on the exact batch (utils/data.py:317-326)."""
        return {"epoch": self.epoch, "batches_consumed": self.batches_consumed,
                "shuffled_indices": self._shuffled_indices.tolist() if self._shuffled_indices is not None else None}

    def load_state_dict(self, state_dict):
        self.epoch = state_dict["epoch"]
        self.batches_consumed = state_dict["batches_consumed"]
        si = state_dict["shuffled_indices"]
        self._shuffled_indices = np.array(si) if si is not None else np.arange(len(self.dataset))
        self._resume_from_state = True

    def shard(self, rank, world_size):
        """Rank `rank`'s interleaved share of the dataset (index i*world+rank, accelerate.py:455)."""
        base = self.dataset

        class _Shard(Dataset):
            def __len__(self_inner):
                return (len(base) + world_size - 1) // world_size

            def __getitem__(self_inner, i):
                return base[(i * world_size + rank) % len(base)]

        return DataLoader(_Shard(), self.batch_size, self.shuffle, self.num_workers, self.prefetch,
                          None if self.collate_fn == self.default_collate else self.collate_fn, self.timeout,
                          self.device, len(self._slots) or 2)
