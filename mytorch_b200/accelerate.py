"""`Accelerator`: mixed precision, gradient accumulation, clipping and
data-parallel gradient sync for the training step — the interface of
mytorch/accelerate.py (GradScaler :31-124, Accelerator :127-1051) over the
CUDA library.

What is laid out differently from the reference, and why:
  * parameters, fp32 masters, gradients and AdamW moments live in FLAT device
    buffers (one per kind); tensors are views at 256-byte-aligned offsets. A
    step is then a handful of launches over whole buffers, the gradient buffer
    is the all-reduce bucket space, and zero_grad is one memset.
  * gradients accumulate in fp32 (the reference accumulates fp16 gradients,
    accelerate.py:716-721); un-scaling, the inf/nan scan, the global norm, the
    clip coefficient, AdamW and the master->half copy read device scalars, so
    the step has NO host synchronisation (the reference syncs once per tensor,
    accelerate.py:724-729, and for the norm, :828).
  * the loss-scale state machine (accelerate.py:91-121) runs in a 1-thread
    kernel; `GradScaler.scale` reads it back only when asked.
  * data parallel: gradients are averaged with NCCL all-reduce over buckets of
    the flat gradient buffer on a side stream (the reference calls all_reduce
    per tensor on temporaries and drops the result, accelerate.py:757-772; the
    intended mean of gradients is what is implemented here). The inf flag and
    the norm are computed AFTER the average, so they agree on every rank
    without extra collectives.
"""
import ctypes as C
import os
import warnings

import numpy as np

from . import _lib
from .array import DeviceArray, stream, synchronize
from .nn.modules import Module
from .optim import Optimizer, TensorTables
from .tensor import Tensor
from .distributed import comm as dist

_ALIGN = 64  # elements: every tensor starts on a 256-byte (fp32) / 128-byte (half) boundary


class GradScaler:
    """Dynamic loss scale (accelerate.py:31-124); the state lives on the device
    as {scale, 1/(scale*accum), clean steps, skipped steps}."""

    def __init__(self, init_scale=2.0 ** 16, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000,
                 dynamic=True, accum_steps=1):
        self.growth_factor, self.backoff_factor, self.growth_interval = growth_factor, backoff_factor, growth_interval
        self.dynamic = dynamic
        self.accum_steps = accum_steps
        self.state = DeviceArray.from_numpy(np.array([init_scale, 1.0 / (init_scale * accum_steps), 0, 0], np.float32))

    @property
    def scale_dev(self):
        return DeviceArray(self.state.ptr, (), "float32", base=self.state)

    @property
    def inv_total_dev(self):
        return DeviceArray(self.state.ptr + 4, (), "float32", base=self.state)

    @property
    def scale(self):          # host read-back (synchronises)
        return float(self.state.numpy()[0])

    @property
    def unskipped(self):
        return int(self.state.numpy()[2])

    @property
    def skipped_steps(self):
        return int(self.state.numpy()[3])

    def update(self, found_inf_dev):
        _lib.scaler_update(self.state.ptr, None if found_inf_dev is None else found_inf_dev.ptr,
                           float(self.growth_factor), float(self.backoff_factor), int(self.growth_interval),
                           1.0 / self.accum_steps, int(self.dynamic), stream())


class _Flat:
    """Flat buffers + per-tensor views for a model's unique parameters."""

    def __init__(self, params, half_dtype):
        self.params = params
        self.offsets, off = [], 0
        for p in params:
            self.offsets.append(off)
            off += (p.data.size + _ALIGN - 1) // _ALIGN * _ALIGN
        self.total = off
        self.master = DeviceArray.zeros((off,), "float32")
        self.grad = DeviceArray.zeros((off,), "float32")
        self.m = DeviceArray.zeros((off,), "float32")
        self.v = DeviceArray.zeros((off,), "float32")
        self.half = DeviceArray.zeros((off,), half_dtype) if half_dtype else None

    def view(self, buf, i, dtype=None):
        p = self.params[i]
        return buf.flat_view(self.offsets[i], p.shape, dtype)


class OptimizerWrapper:
    """Gates step/zero_grad on the accumulation counter (accelerate.py:342-378)."""

    def __init__(self, optimizer, accelerator):
        self.optimizer, self.acc = optimizer, accelerator

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def step(self):
        a = self.acc
        if a.step_counter % a.gradient_accumulation_steps != 0:
            return
        a._finish_gradients()
        self.optimizer.fused_ctx = a._fused_ctx()
        self.optimizer.step()
        a.scaler.update(a._found_inf)
        a._grads_ready = False

    def zero_grad(self):
        a = self.acc
        if a.step_counter % a.gradient_accumulation_steps != 0:
            return
        a._flat.grad.zero_()
        a._max_norm = 0.0

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, sd):
        return self.optimizer.load_state_dict(sd)

    def __repr__(self):
        return f"OptimizerWrapper({self.optimizer.__class__.__name__})"


class Accelerator:
    def __init__(self, num_gpus=None, rank=None, gradient_accumulation_steps=1, mixed_precision=False,
                 log_wandb=False, master_addr=None, master_port=None, half_dtype="float16", bucket_mb=64,
                 overlap_comm=True):
        self.rank = rank if rank is not None else int(os.environ.get("RANK", 0))
        self.world_size = num_gpus if num_gpus is not None else int(os.environ.get("WORLD_SIZE", 1))
        self.local_rank = int(os.environ.get("LOCAL_RANK", self.rank))
        self.master_addr = master_addr or os.environ.get("CUPYX_DISTRIBUTED_HOST") or os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = master_port or os.environ.get("CUPYX_DISTRIBUTED_PORT")
        if port is None:
            port = int(os.environ.get("MASTER_PORT", "13332")) + 1   # torchrun owns MASTER_PORT itself
        self.master_port = int(port)
        _lib.require_device()
        _lib.set_device(self.local_rank % max(1, _lib.device_count()))
        self.gradient_accumulation_steps = gradient_accumulation_steps
        self.step_counter = 0
        self.comm = None
        if self.world_size > 1:
            self.comm = dist.NCCLBackend(self.world_size, self.rank, self.master_addr, self.master_port)
        np.random.seed(42 + self.rank)
        env_val = os.environ.get("MYTORCHRUN_MIXED_PRECISION", False)
        self.mixed_precision = mixed_precision if env_val is False else (env_val != "No")
        self.half_dtype = half_dtype
        self.skip_optimizer_step = False
        # fp32 and bf16 runs keep a fixed scale of 1; fp16 uses the dynamic scale
        dynamic = bool(self.mixed_precision) and half_dtype == "float16"
        self.scaler = GradScaler(init_scale=2.0 ** 16 if dynamic else 1.0, dynamic=dynamic,
                                 accum_steps=gradient_accumulation_steps)
        # backward() hands this device scalar to loss.backward(); a loss that computes its gradient
        # in the forward pass (F.cross_entropy(..., fused_backward=True)) folds it in right there
        Tensor.loss_grad_hint = self.scaler.scale_dev
        self._scalars = DeviceArray.zeros((4,), "float32")    # [sumsq, found_inf, -, -]
        self._sumsq = DeviceArray(self._scalars.ptr, (), "float32", base=self._scalars)
        self._found_inf = DeviceArray(self._scalars.ptr + 4, (), "float32", base=self._scalars)
        self._max_norm = 0.0
        self._grads_ready = False
        self._grad_tables = None
        self._flat = None
        self.bucket_elems = bucket_mb * 1024 * 1024 // 4
        self.overlap_comm = overlap_comm
        self.model = None
        self.wandb_enabled = False

    # ---- bookkeeping identical to the reference ----
    def is_main_process(self):
        return self.rank == 0

    def print(self, *a, **k):
        if self.rank == 0:
            print(*a, **k)

    @property
    def device(self):
        return f"cuda:{self.local_rank}"

    @property
    def num_processes(self):
        return self.world_size

    @property
    def sync_grad(self):
        return self.step_counter % self.gradient_accumulation_steps == 0

    @property
    def grad_norm(self):
        """Global gradient norm of the last completed step (host read-back)."""
        return float(np.sqrt(self._sumsq.numpy()))

    def prepare(self, *args):
        out = []
        for obj in args:
            if isinstance(obj, Module):
                out.append(self.prepare_model(obj))
            elif isinstance(obj, Optimizer):
                out.append(self.prepare_optimizer(obj))
            else:
                out.append(self.prepare_dataloaders(obj))
        return out

    # ---- model: flat buffers, masters, half copies, broadcast (accelerate.py:242-290) ----
    def prepare_model(self, model):
        self.model = model
        params = model.parameters()                      # unique (tied weights once)
        flat = _Flat(params, self.half_dtype if self.mixed_precision else None)
        self._masters = []
        for i, p in enumerate(params):
            mview = flat.view(flat.master, i)
            _lib.cast(p.data.ptr, p.data.code, mview.ptr, mview.code, p.data.size, stream())
        if self.comm is not None:
            self.comm.broadcast(flat.master, root=0)
        for i, p in enumerate(params):
            mview = flat.view(flat.master, i)
            gview = flat.view(flat.grad, i)
            if self.mixed_precision:
                hview = flat.view(flat.half, i)
                _lib.cast(mview.ptr, mview.code, hview.ptr, hview.code, mview.size, stream())
                master = Tensor(mview, requires_grad=True)
                master.is_param = True
                master.grad = gview
                self._masters.append(master)
                p.data = hview                            # the model now computes in half precision
            else:
                p.data = mview
                self._masters.append(p)
            p.grad = gview                                # persistent fp32 accumulation view
        self._flat = flat
        self._param_index = {id(p): i for i, p in enumerate(params)}
        # id(model parameter) -> (offset, count) in the flat gradient buffer, for bucket triggering
        self._param_ranges = {id(p): (flat.offsets[i], p.data.size) for i, p in enumerate(params)}
        wd = [0.0] * len(params)
        self._grad_tables = TensorTables([flat.view(flat.master, i) for i in range(len(params))],
                                         [flat.view(flat.grad, i) for i in range(len(params))], None, None, None, wd)
        return model

    # ---- optimizer: re-point groups at the masters and the flat moments (accelerate.py:292-386) ----
    def prepare_optimizer(self, optimizer):
        flat = self._flat
        assert flat is not None, "prepare the model before the optimizer"
        for group in optimizer.param_groups:
            idx = [self._param_index[id(p)] for p in group["params"]]
            group["params"] = [self._masters[i] for i in idx]
            group["m"] = [flat.view(flat.m, i) for i in idx]
            group["v"] = [flat.view(flat.v, i) for i in idx]
            group["_tables"] = None
        self._half_map = {}
        if self.mixed_precision:
            for i in range(len(flat.params)):
                self._half_map[flat.view(flat.master, i).ptr] = flat.view(flat.half, i)
        self.optimizer = optimizer
        return OptimizerWrapper(optimizer, self)

    def prepare_dataloaders(self, loader):
        """Shards an indexable dataset across ranks by interleaving
        (idx * world + rank, accelerate.py:455); other objects pass through."""
        if self.world_size > 1 and hasattr(loader, "shard"):
            loader = loader.shard(self.rank, self.world_size)
        if hasattr(loader, "state_dict") and hasattr(loader, "load_state_dict"):
            # prepared loaders are checkpointed with the rest of the state (accelerate.py:970-976)
            if not hasattr(self, "dataloaders"):
                self.dataloaders = []
            self.dataloaders.append(loader)
        return loader

    def _fused_ctx(self):
        return {"p_half": self._half_map or None, "inv_scale": self.scaler.inv_total_dev.ptr,
                "sumsq": self._sumsq.ptr, "max_norm": self._max_norm, "found_inf": self._found_inf.ptr}

    # ---- backward (accelerate.py:675-797) ----
    def backward(self, loss):
        """Scaled backward of one micro-batch. The upstream gradient is the
        device-resident loss scale; nothing is read back."""
        g = self.scaler.scale_dev
        last_micro = (self.step_counter + 1) % self.gradient_accumulation_steps == 0
        if self.comm is not None and last_micro and self.overlap_comm:
            # gradients become final during this backward: reduce them bucket by bucket as they do
            self.comm.begin_overlap(self._flat.grad, self.bucket_elems, self._param_ranges)
            Tensor.param_ready_hook = self.comm.param_ready
        try:
            loss.backward(g)
        finally:
            Tensor.param_ready_hook = None
        self.step_counter += 1
        if self.step_counter % self.gradient_accumulation_steps == 0:
            self._grads_ready = False
            self._finish_gradients()

    def _finish_gradients(self):
        """On an accumulation boundary: average across ranks, then the inf/nan
        flag and the sum of squares of the un-scaled gradients (device scalars)."""
        if self._grads_ready:
            return
        if self.comm is not None:
            if self.comm._ov_active:
                self.comm.finish_overlap()
            else:
                self.comm.allreduce_grads(self._flat.grad, self.bucket_elems)
        t = self._grad_tables
        _lib.gradnorm_multi(C.byref(t.c), _lib.F32, self.scaler.inv_total_dev.ptr, self._sumsq.ptr,
                            self._found_inf.ptr, stream())
        self._grads_ready = True

    def clip_grad_norm_(self, max_norm=1.0):
        """Global-norm clipping (accelerate.py:799-856). The coefficient
        min(1, max_norm / (norm + 1e-6)) is applied inside the fused AdamW
        kernel from the device-side norm, so gradients are not rewritten."""
        if self.step_counter % self.gradient_accumulation_steps != 0:
            return None
        self._finish_gradients()
        self._max_norm = float(max_norm)
        return None

    # ---- metrics (accelerate.py:858-880) ----
    def gather_for_metrics(self, value):
        assert isinstance(value, Tensor) and value.shape == (), "value must be a scalar Tensor"
        if self.comm is None:
            return value
        out = DeviceArray.empty((), "float32")
        self.comm.all_reduce(value.data.astype("float32"), out, op="avg")
        return Tensor(out)

    def wait_for_everyone(self):
        if self.comm is not None:
            self.comm.barrier()

    def end_training(self):
        if self.comm is not None:
            self.comm.barrier()
            self.comm.stop()
            self.comm = None

    # ---- checkpoint, same files and layouts as the reference (accelerate.py:916-1048) ----
    #   model.safetensors  fp32 master of every parameter, keyed by _named_parameters_no_dedup
    #   optimizer.bin      pickled AdamW.state_dict()
    #   mp_config.bin      pickled {scale, growth_factor, backoff_factor, growth_interval, unskipped}
    #   dataloader_{i}.bin pickled state_dict() of the i-th prepared loader (epoch, batches consumed,
    #                      shuffled order), so a resumed run continues on the next batch
    # so a run can move between the two implementations mid-training.
    def save_state(self, path_to_checkpoint, save_model_only=False):
        import pickle
        from safetensors.numpy import save_file
        if self.rank == 0:
            os.makedirs(path_to_checkpoint, exist_ok=True)
            if self.model is not None:
                sd = {}
                for name, p in self.model._named_parameters_no_dedup():
                    i = self._param_index.get(id(p))
                    a = self._flat.view(self._flat.master, i).numpy() if i is not None else p.numpy()
                    sd[name] = np.ascontiguousarray(a, dtype=np.float32)
                save_file(sd, os.path.join(path_to_checkpoint, "model.safetensors"))
            if not save_model_only:
                if getattr(self, "optimizer", None) is not None:
                    with open(os.path.join(path_to_checkpoint, "optimizer.bin"), "wb") as fh:
                        pickle.dump(self.optimizer.state_dict(), fh)
                if self.mixed_precision:
                    st = self.scaler.state.numpy()
                    cfg = {"scale": float(st[0]), "growth_factor": self.scaler.growth_factor,
                           "backoff_factor": self.scaler.backoff_factor, "growth_interval": self.scaler.growth_interval,
                           "unskipped": int(st[2])}
                    with open(os.path.join(path_to_checkpoint, "mp_config.bin"), "wb") as fh:
                        pickle.dump(cfg, fh)
                for idx, loader in enumerate(getattr(self, "dataloaders", [])):
                    with open(os.path.join(path_to_checkpoint, f"dataloader_{idx}.bin"), "wb") as fh:
                        pickle.dump(loader.state_dict(), fh)
        self.wait_for_everyone()

    def load_state(self, path_to_checkpoint):
        import pickle
        import warnings
        from safetensors.numpy import load_file
        path_to_model = os.path.join(path_to_checkpoint, "model.safetensors")
        if os.path.exists(path_to_model) and self.model is not None:
            sd = load_file(path_to_model)
            for name, p in self.model._named_parameters_no_dedup():
                i = self._param_index.get(id(p))
                if i is None:
                    continue
                mview = self._flat.view(self._flat.master, i)
                mview.set_from_numpy(np.asarray(sd[name], dtype=np.float32).reshape(mview.shape))
                if self.mixed_precision:
                    hview = self._flat.view(self._flat.half, i)
                    _lib.cast(mview.ptr, mview.code, hview.ptr, hview.code, mview.size, stream())
            if self.comm is not None:          # every rank starts from rank 0's weights
                self.comm.broadcast(self._flat.master, root=0)
                if self.mixed_precision:
                    self.comm.broadcast(self._flat.half, root=0)
        path_to_optimizer = os.path.join(path_to_checkpoint, "optimizer.bin")
        if os.path.exists(path_to_optimizer) and getattr(self, "optimizer", None) is not None:
            with open(path_to_optimizer, "rb") as fh:
                self.optimizer.load_state_dict(pickle.load(fh))
        if self.mixed_precision:
            path_to_mp = os.path.join(path_to_checkpoint, "mp_config.bin")
            if os.path.exists(path_to_mp):
                with open(path_to_mp, "rb") as fh:
                    cfg = pickle.load(fh)
                self.scaler.growth_factor = cfg["growth_factor"]
                self.scaler.backoff_factor = cfg["backoff_factor"]
                self.scaler.growth_interval = cfg["growth_interval"]
                st = self.scaler.state.numpy()
                st[0] = cfg["scale"]
                st[1] = 1.0 / (cfg["scale"] * self.scaler.accum_steps)
                st[2] = cfg["unskipped"]
                self.scaler.state.set_from_numpy(st)
            else:
                warnings.warn("If you are resuming mixed precision training without its checkpointed config, "
                              "you may have instability in training")
        for idx, loader in enumerate(getattr(self, "dataloaders", [])):
            path_to_loader = os.path.join(path_to_checkpoint, f"dataloader_{idx}.bin")
            if os.path.exists(path_to_loader):
                with open(path_to_loader, "rb") as fh:
                    loader.load_state_dict(pickle.load(fh))
            else:
                warnings.warn(f"Couldn't find {path_to_loader}, cannot resume dataloader, starting from scratch!!")
