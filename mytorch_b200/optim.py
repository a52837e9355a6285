"""AdamW and the cosine schedule of the reference optimiser package
(mytorch/optim/optimizers.py:288-455, mytorch/optim/lr_scheduler.py:60-90).

Same constructor, `param_groups` layout and update rule as the reference —
decay applied AFTER the Adam update, eps not bias-corrected
(optimizers.py:342-371) — but one kernel launch per parameter group instead of
~12 elementwise launches per tensor: pointer/size/chunk tables are built once
on the device and `mt_adamw_multi` walks every tensor of the group.
"""
import ctypes as C
import math

import numpy as np

from . import _lib
from .array import DeviceArray, stream

_CHUNK = 4096


class TensorTables:
    """Device-side description of a list of tensors for the multi-tensor
    kernels (see mt_tensor_list in the C header)."""

    def __init__(self, p, g, m, v, p_half, weight_decay):
        n = len(p)
        self.keep = (p, g, m, v, p_half)
        sizes = np.array([a.size for a in p], dtype=np.int64)
        chunk_tensor, chunk_offset = [], []
        for i, s in enumerate(sizes):
            offs = np.arange(0, s, _CHUNK, dtype=np.int64)
            chunk_tensor.append(np.full(len(offs), i, dtype=np.int32))
            chunk_offset.append(offs)
        ct = np.concatenate(chunk_tensor) if n else np.zeros(0, np.int32)
        co = np.concatenate(chunk_offset) if n else np.zeros(0, np.int64)

        def ptrs(arrs):
            return DeviceArray.from_numpy(np.array([0 if a is None else a.ptr for a in arrs], dtype=np.int64), "int64")
        self.dev = dict(p=ptrs(p), g=ptrs(g), m=ptrs(m) if m else None, v=ptrs(v) if v else None,
                        p_half=ptrs(p_half) if p_half else None,
                        size=DeviceArray.from_numpy(sizes, "int64"),
                        wd=DeviceArray.from_numpy(np.asarray(weight_decay, dtype=np.float32)),
                        ct=DeviceArray.from_numpy(ct, "int32"), co=DeviceArray.from_numpy(co, "int64"))
        d = self.dev
        self.c = _lib.TensorList(d["p"].ptr, d["g"].ptr, d["m"].ptr if m else None, d["v"].ptr if v else None,
                                 d["p_half"].ptr if p_half else None, d["size"].ptr, d["wd"].ptr,
                                 d["ct"].ptr, d["co"].ptr, n, len(ct))
        self.g_dtype = g[0].dtype if n else "float32"
        self.half_dtype = next((a.dtype for a in (p_half or []) if a is not None), "float16")
        self.key = tuple(a.ptr for a in p) + tuple(a.ptr for a in g)


class Optimizer:
    pass


class AdamW(Optimizer):
    def __init__(self, parameters, lr=0.001, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
        parameters = list(parameters)
        if parameters and isinstance(parameters[0], dict):
            self.param_groups = [{
                "params": [p for p in g["params"] if p.requires_grad],
                "lr": g.get("lr", lr), "beta1": g.get("beta1", beta1), "beta2": g.get("beta2", beta2),
                "eps": g.get("eps", eps), "weight_decay": g.get("weight_decay", weight_decay)} for g in parameters]
        else:
            self.param_groups = [{"params": [p for p in parameters if p.requires_grad], "lr": lr, "beta1": beta1,
                                  "beta2": beta2, "eps": eps, "weight_decay": weight_decay}]
        self._init_optimizer_state()
        # set by Accelerator for mixed precision / clipping: device scalars and half copies
        self.fused_ctx = None

    def _init_optimizer_state(self, device="cuda"):
        for group in self.param_groups:
            group["m"] = [DeviceArray.zeros(p.shape, "float32") for p in group["params"]]
            group["v"] = [DeviceArray.zeros(p.shape, "float32") for p in group["params"]]
            group["_tables"] = None
            self._set_step_state(group, 0, 1.0, 1.0)

    # The step count and the running beta powers are device scalars (two slots of doubles, see
    # mt_adamw_multi): a step that the loss-scale logic skips on the device must not advance them
    # (the reference does not call optimizer.step() on an overflow, mytorch/accelerate.py:342-352),
    # and the host never learns about a skip without a read-back.
    @staticmethod
    def _set_step_state(group, t, b1p, b2p):
        host = np.array([t, b1p, b2p, 0.0] * 2, dtype=np.float64)
        group["_step_state"] = DeviceArray.from_numpy(host.view(np.int64), "int64")
        group["_slot"] = 0

    @staticmethod
    def _get_step_state(group):
        host = group["_step_state"].numpy().view(np.float64).reshape(2, 4)[group["_slot"]]
        return int(round(host[0])), float(host[1]), float(host[2])

    def _tables(self, group):
        ctx = self.fused_ctx or {}
        halves = ctx.get("p_half")
        idx = [i for i, p in enumerate(group["params"]) if p.grad is not None]
        p = [group["params"][i].data for i in idx]
        g = [group["params"][i].grad for i in idx]
        key = tuple(a.ptr for a in p) + tuple(a.ptr for a in g)
        t = group.get("_tables")
        if t is None or t.key != key:
            ph = [halves.get(group["params"][i].data.ptr) for i in idx] if halves else None
            t = TensorTables(p, g, [group["m"][i] for i in idx], [group["v"][i] for i in idx], ph,
                             [group["weight_decay"]] * len(idx))
            group["_tables"] = t
        return t

    def step(self):
        ctx = self.fused_ctx or {}
        for group in self.param_groups:
            t = self._tables(group)
            if t.c.n_tensors == 0:
                continue
            _lib.adamw_multi(C.byref(t.c), _lib.F32 if t.g_dtype == "float32" else (_lib.F16 if t.g_dtype == "float16" else _lib.BF16),
                             _lib.F16 if t.half_dtype == "float16" else _lib.BF16,
                             float(group["lr"]), float(group["beta1"]), float(group["beta2"]),
                             float(group["eps"]), ctx.get("inv_scale"), ctx.get("sumsq"), float(ctx.get("max_norm", 0.0)),
                             ctx.get("found_inf"), 0, group["_step_state"].ptr, group["_slot"], stream())
            group["_slot"] ^= 1

    def zero_grad(self):
        for group in self.param_groups:
            for p in group["params"]:
                p.grad = None

    def state_dict(self):
        """Same layout as the reference's AdamW.state_dict (optimizers.py:378-407):
        {"state": [per group {m, v, t, beta1_pow, beta2_pow}], "param_groups": [per group
        {lr, beta1, beta2, eps, weight_decay, num_params}]}; the moments are host NumPy arrays."""
        sd = {"state": [], "param_groups": []}
        for g in self.param_groups:
            t, b1p, b2p = self._get_step_state(g)
            sd["state"].append({"m": [a.numpy() for a in g["m"]], "v": [a.numpy() for a in g["v"]],
                                "t": t, "beta1_pow": b1p, "beta2_pow": b2p})
            sd["param_groups"].append({"lr": g["lr"], "beta1": g["beta1"], "beta2": g["beta2"], "eps": g["eps"],
                                       "weight_decay": g["weight_decay"], "num_params": len(g["params"])})
        return sd

    def load_state_dict(self, sd):
        """Accepts the layout above (optimizers.py:410-441). Moments may be NumPy arrays or any
        object that wraps one (`_array` attribute, `.get()` for device arrays, `__array__`)."""
        if len(sd["state"]) != len(self.param_groups):
            raise ValueError(f"Loaded state dict has {len(sd['state'])} parameter groups, "
                             f"but optimizer has {len(self.param_groups)} parameter groups")

        def host(a):
            a = getattr(a, "_array", a)
            if hasattr(a, "get") and not isinstance(a, np.ndarray):
                a = a.get()
            return np.asarray(a, dtype=np.float32)

        for i, (g, st) in enumerate(zip(self.param_groups, sd["state"])):
            if len(g["params"]) != len(st["m"]):
                raise ValueError(f"Parameter group {i}: loaded state has {len(st['m'])} parameters, "
                                 f"but optimizer has {len(g['params'])} parameters")
            for a, h in zip(g["m"], st["m"]):
                a.set_from_numpy(host(h).reshape(a.shape))
            for a, h in zip(g["v"], st["v"]):
                a.set_from_numpy(host(h).reshape(a.shape))
            self._set_step_state(g, st["t"], st["beta1_pow"], st["beta2_pow"])
            lg = sd["param_groups"][i]
            for k in ("lr", "beta1", "beta2", "eps", "weight_decay"):
                g[k] = lg[k]


class CosineLRScheduler:
    """Linear warm-up then cosine decay, written into every group's "lr" on
    each step() (mytorch/optim/lr_scheduler.py:60-90). As in the reference the
    optimizer keeps its constructor lr until the first step()."""

    def __init__(self, optimizer, max_lr, min_lr=0.0, total_steps=1000, warmup_steps=0):
        self.optimizer, self.max_lr, self.min_lr = optimizer, max_lr, min_lr
        self.total_steps, self.warmup_steps = total_steps, warmup_steps
        self.step_count = 0

    def step(self):
        self.step_count += 1
        if self.step_count <= self.warmup_steps:
            lr = self.max_lr * self.step_count / self.warmup_steps
        else:
            progress = (self.step_count - self.warmup_steps) / max(1, self.total_steps - self.warmup_steps)
            lr = self.min_lr + 0.5 * (self.max_lr - self.min_lr) * (1 + math.cos(math.pi * progress))
        for g in self.optimizer.param_groups:
            g["lr"] = lr
        return lr
