"""Benchmark of the GPT training step (tokens/s and MFU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config gpt2|d20]

Own arm: one process per GPU (torchrun-style env for N > 1). A step is one
optimizer step: forward + backward of `accum` micro-batches, gradient all-reduce
(N > 1), global-norm clip, fused AdamW with fp16 dynamic loss scaling.
  --config gpt2 (default): GPT-2 124M, micro-batch 16 x 1024 tokens. N = 1 runs the
      single-GPU configuration (accum = 1); N > 1 the data-parallel one (global batch
      524288 tokens, accum = 32 / N).
  --config d20: the nanochat-style d20 model (L20 d1280 10x128 heads ctx2048 vocab65536,
      rotary + QK-norm, ReLU^2, untied head), micro-batch 32 x 2048 tokens per GPU, global
      batch 524288 tokens at N = 8 (accum = 8 / N for N > 1, 1 at N = 1).
Timing: CUDA events on the compute stream around exactly K steps, bracketed by barrier +
synchronize, max over ranks. `value` has the token ids resident in HBM; `e2e` repeats the K
steps with host batches: every step copies its ids and labels from pinned host memory to the
device and its loss from the device to pinned host memory, and the host reads every loss inside
the timed region - one step late (it waits for step n - 1's copy after queueing step n), the
last one before the closing event.

Reference arm (`--impl reference`): the reference's algorithm for the same step on the host
cores (the NumPy oracle, which is pinned to the reference by the golden vectors), with every
host thread, on a bounded sample of the workload: the full model, one short sequence per step.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(vocab_size=50304, max_seq_len=1024, embed_dim=768, mlp_ratio=4, num_blocks=12, num_heads=12)
MICRO_B, CTX, VOCAB_DATA = 16, 1024, 50257
GLOBAL_TOKENS = 524288
LR, WD, CLIP = 6e-4, 0.1, 1.0

D20_CFG = dict(vocab_size=65536, max_seq_len=2048, embed_dim=1280, mlp_ratio=4, num_blocks=20,
               num_q_heads=10, num_kv_heads=10)

WORKLOADS = {
    "gpt2": dict(metric="GPT-2 124M train tokens/s", cfg=CFG, micro_b=MICRO_B, ctx=CTX, vocab_data=VOCAB_DATA,
                 lr=LR, wd=WD, clip=CLIP, ref_tokens=1024,
                 label="GPT-2 124M (L12 H12 d768 ctx1024 vocab50304, tied) fp16 mixed precision, "
                       "AdamW lr6e-4 wd0.1 clip1.0, micro-batch 16x1024",
                 l2="working set per step (>2 GB of activations, 1.6 GB logits) exceeds the 126 MB L2"),
    "d20": dict(metric="nanochat d20 train tokens/s", cfg=D20_CFG, micro_b=32, ctx=2048, vocab_data=65536,
                lr=3e-4, wd=0.1, clip=1.0, ref_tokens=256,
                label="nanochat-style d20 (L20 d1280 10x128 heads ctx2048 vocab65536, rotary + QK-norm, ReLU^2, "
                      "untied head, soft-capped loss) fp16 mixed precision, AdamW lr3e-4 wd0.1 clip1.0, "
                      "micro-batch 32x2048",
                l2="working set per step (>60 GB of activations, 8.6 GB logits) exceeds the 126 MB L2"),
}


def flops_per_token(cfg=CFG, ctx=CTX):
    """fwd+bwd model FLOPs per token, causal-exact attention: 6*P_mm + 6*L*T*d. P_mm counts every
    weight that takes part in a matmul (the four attention projections, the two MLP matrices,
    the lm_head); an embedding lookup is not a matmul."""
    d, L = cfg["embed_dim"], cfg["num_blocks"]
    p_mm = L * (3 * d * d + d * d + 2 * cfg["mlp_ratio"] * d * d) + d * cfg["vocab_size"]
    return 6 * p_mm + 6 * L * ctx * d


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            p = json.load(fh)
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops_sustained"], "source": "measured (sustained)"}
    except Exception:
        return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback"}


def gemm_capture():
    """DRAM traffic of one captured GEMM launch and the same-data library figure: quantities of a
    profiler capture, kept as data next to the summary they come from."""
    try:
        with open(os.path.join(ROOT, "profiles", "gemm_capture.json")) as fh:
            return json.load(fh)
    except Exception:
        return {}


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([time.perf_counter()] + [c.strip() for c in line.split(",")])

    def summary(self, window=None):
        """Summary of the samples taken inside `window` = (t0, t1) in perf_counter seconds (all
        samples when none fell inside it)."""
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = list(self.rows)
        if window is not None:
            inside = [r for r in rows if window[0] <= r[0] <= window[1]]
            rows = inside or rows
        for r in (row[1:] for row in rows):
            try:
                sm.append(float(r[1])); mx.append(float(r[2])); pw.append(float(r[3]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w": float(np.median(pw)) if pw else None, "reasons": sorted(reasons), "samples": len(sm)}

    def stop(self, window=None):
        if self.proc is not None:
            self.proc.terminate()      # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        return self.summary(window)


# --------------------------------------------------------------- reference arm ----
def _all_host_threads():
    """A launcher may export OMP_NUM_THREADS=1 (torchrun does); the CPU arm is meant to use every
    host core, so the BLAS pool is sized explicitly."""
    try:
        from threadpoolctl import threadpool_limits
        return threadpool_limits(limits=os.cpu_count() or 1)
    except Exception:
        import contextlib
        return contextlib.nullcontext()


def _oracle_step_fn(w):
    """One optimizer step of the NumPy oracle on one sequence of w["ref_tokens"] tokens of the
    full model; returns (step function, description of the sample)."""
    from oracle import gpt2 as og
    from oracle import ops as O
    T = w["ref_tokens"]
    if w is WORKLOADS["gpt2"]:
        cfg = og.GPT2Config(**w["cfg"])
        params = og.init_params(cfg, seed=0)
        fwd, bwd = og.forward, og.backward
    else:
        from oracle import nanochat as on
        c = w["cfg"]
        cfg = on.GPTConfig(vocab_size=c["vocab_size"], max_seq_len=c["max_seq_len"], embed_dim=c["embed_dim"],
                           mlp_ratio=c["mlp_ratio"], num_blocks=c["num_blocks"], num_heads=c["num_q_heads"])
        params = on.init_params(cfg, seed=0)
        fwd = lambda p, cf, x, y: (lambda r: (r[0], None, r[-1]))(on.forward(p, cf, x, y))
        bwd = on.backward
    opt = og.AdamW(params, w["lr"], 0.9, 0.95, 1e-8, w["wd"])
    rng = np.random.default_rng(0)

    def step():
        x, y = og.synthetic_batch(rng, 1, T, w["vocab_data"])
        _, _, cache = fwd(params, cfg, x, y)
        grads = bwd(params, cfg, cache)
        O.clip_grad_norm(list(grads.values()), w["clip"])
        opt.step(params, grads)
    sample = (f"full model, 1 sequence x {T} tokens per step (of {w['micro_b']} x {w['ctx']}), fp32 NumPy oracle")
    return step, sample, T


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    w = WORKLOADS[args.config]
    cores = os.cpu_count() or 1
    with _all_host_threads():
        step, sample, T = _oracle_step_fn(w)
        times = []
        for i in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            step()
            if i >= args.warmup:
                times.append(time.perf_counter() - t0)
    sec = float(np.mean(times))
    val = T / sec
    print(json.dumps({
        "impl": "reference", "metric": w["metric"], "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.gpus, accum_for(args.gpus, args.config), args.config),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_baseline_sample(config="gpt2", seconds_budget=30.0):
    """The oracle's step on a bounded sample (one short sequence, full model), one timed step
    after one warm-up, or just the warm-up if that already took long."""
    w = WORKLOADS[config]
    with _all_host_threads():
        step, sample, T = _oracle_step_fn(w)
        times = []
        for i in range(2):
            t0 = time.perf_counter()
            step()
            times.append(time.perf_counter() - t0)
            if times[-1] > seconds_budget / 2:
                break
    return {"value": T / times[-1], "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"{sample}, {len(times)} step(s), last timed"}


def accum_for(n_gpus, config="gpt2"):
    w = WORKLOADS[config]
    return 1 if n_gpus == 1 else max(1, GLOBAL_TOKENS // (w["micro_b"] * w["ctx"] * n_gpus))


def config_dict(n_gpus, accum, config="gpt2"):
    w = WORKLOADS[config]
    tokens = w["micro_b"] * w["ctx"] * n_gpus * accum
    return {"workload": w["label"] + ("" if n_gpus == 1 else f", DDP global batch {tokens} tokens"),
            "micro_batch": w["micro_b"], "seq_len": w["ctx"], "grad_accum": accum,
            "global_batch_tokens": tokens, "parallelism": f"dp{n_gpus}", "l2": w["l2"]}


# ------------------------------------------------------------------- own arm ----
def run_own(args):
    import mytorch_b200 as mt
    from mytorch_b200 import _lib
    from mytorch_b200.array import DeviceArray, stream
    from mytorch_b200.tensor import no_grad

    w = WORKLOADS[args.config]
    micro_b, ctx, vocab_data, clip = w["micro_b"], w["ctx"], w["vocab_data"], w["clip"]
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")
    accum = accum_for(world, args.config)
    if args.gemm_tile_policy:
        _lib.gemm_tile_policy(args.gemm_tile_policy)
    acc = mt.Accelerator(num_gpus=world, rank=rank, gradient_accumulation_steps=accum, mixed_precision=True)
    np.random.seed(1234)                      # identical initial weights on every rank
    if args.config == "gpt2":
        from mytorch_b200.gpt2 import GPT2, GPT2Config
        model = GPT2(GPT2Config(**w["cfg"]))
        # the training loop never looks at the logits after the loss: let the loss overwrite them with
        # their gradient in its forward pass (one read + one write of the 1.65 GB instead of 2 + 1)
        loss_fn = mt.nn.CrossEntropyLoss(fused_backward=True)
        forward_loss = lambda x, y: loss_fn(model(mt.Tensor(x)), mt.Tensor(y))
    else:
        from mytorch_b200.nanochat_gpt import GPT, GPTConfig
        model = GPT(GPTConfig(**w["cfg"]))
        # the model zero-initialises out_proj and lm_head (nanochat_gpt.py:287-288); a step on zeros
        # multiplies zeros in a quarter of the GEMMs, which a power-capped board runs faster than
        # real data, so the benchmark gives them the other Linear layers' initialisation
        for name, p in model.named_parameters():
            if ("out_proj" in name) or ("lm_head" in name):
                fan_out, fan_in = p.shape
                std = 1.0 / np.sqrt(fan_in) * min(1.0, np.sqrt(fan_out / fan_in))
                p.data.set_from_numpy((np.random.randn(*p.shape) * std).astype(np.float32))
        model.loss_mode = args.loss_mode
        forward_loss = lambda x, y: model(mt.Tensor(x), mt.Tensor(y))[1]
    decay, no_decay = [], []
    for _, p in model.named_parameters():
        (no_decay if len(p.shape) < 2 else decay).append(p)
    groups = [{"params": decay, "weight_decay": w["wd"]}]
    if no_decay:
        groups.append({"params": no_decay, "weight_decay": 0.0})
    opt = mt.optim.AdamW(groups, lr=w["lr"], beta1=0.9, beta2=0.95)
    model, opt = acc.prepare(model, opt)
    if acc.comm is not None:
        acc.comm.record_exposed = True

    rng = np.random.default_rng(100 + rank)
    n_batches = 4
    host_ids = [rng.integers(0, vocab_data, (micro_b, ctx + 1)) for _ in range(n_batches)]
    dev_x = [DeviceArray.from_numpy(h[:, :-1].astype(np.int32)) for h in host_ids]
    dev_y = [DeviceArray.from_numpy(h[:, 1:].astype(np.int32)) for h in host_ids]

    # pinned host staging for the end-to-end pass
    nbytes = micro_b * ctx * 4
    pin = C.c_void_p()
    _lib.host_alloc(C.byref(pin), 2 * nbytes * n_batches + 64)
    pinned = np.ctypeslib.as_array((C.c_int32 * (2 * micro_b * ctx * n_batches)).from_address(pin.value))
    for i, h in enumerate(host_ids):
        pinned[(2 * i) * micro_b * ctx:(2 * i + 1) * micro_b * ctx] = h[:, :-1].reshape(-1)
        pinned[(2 * i + 1) * micro_b * ctx:(2 * i + 2) * micro_b * ctx] = h[:, 1:].reshape(-1)
    stage_x = DeviceArray.empty((micro_b, ctx), "int32")
    stage_y = DeviceArray.empty((micro_b, ctx), "int32")
    loss_pin = C.c_void_p()
    _lib.host_alloc(C.byref(loss_pin), 64)
    loss_host = np.ctypeslib.as_array((C.c_float * 16).from_address(loss_pin.value))
    loss_events = [C.c_void_p(), C.c_void_p()]
    for ev in loss_events:
        _lib.event_create(C.byref(ev))
    e2e_state = {"n": 0, "last": None}

    counter = [0]

    def micro(x, y):
        loss = forward_loss(x, y)
        acc.backward(loss)
        acc.clip_grad_norm_(clip)
        opt.step()
        opt.zero_grad()
        return loss

    def step_resident():
        for _ in range(acc.gradient_accumulation_steps):
            i = counter[0] % n_batches
            counter[0] += 1
            loss = micro(dev_x[i], dev_y[i])
        return loss

    def step_e2e():
        """One optimizer step fed from pinned host memory, its loss copied back to pinned host
        memory. The host reads each step's loss one step late - it waits for the copy of step n - 1
        after it has queued step n - the way a training loop logs its loss without draining the
        GPU; e2e_drain() reads the last one. Every step's loss is read inside the timed region."""
        for _ in range(acc.gradient_accumulation_steps):
            i = counter[0] % n_batches
            counter[0] += 1
            base = pin.value + (2 * i) * nbytes
            _lib.memcpy_h2d(stage_x.ptr, base, nbytes, stream())
            _lib.memcpy_h2d(stage_y.ptr, base + nbytes, nbytes, stream())
            loss = micro(stage_x, stage_y)
        n = e2e_state["n"]
        _lib.memcpy_d2h(loss_pin.value + 4 * (n & 1), loss.data.ptr, 4, stream())
        _lib.event_record(loss_events[n & 1], stream())
        if n > 0:
            _lib.event_sync(loss_events[(n - 1) & 1])
            e2e_state["last"] = float(loss_host[(n - 1) & 1])
        e2e_state["n"] = n + 1
        return loss

    def e2e_drain():
        n = e2e_state["n"]
        if n > 0:
            _lib.event_sync(loss_events[(n - 1) & 1])
            e2e_state["last"] = float(loss_host[(n - 1) & 1])
        e2e_state["n"] = 0

    def barrier():
        if acc.comm is not None:
            acc.comm.barrier()
        _lib.device_sync()

    host_ms = [0.0]
    window = [0.0, 0.0]      # host time of the last timed region, for the clock samples

    def timed(fn, steps, after=None):
        e0, e1 = C.c_void_p(), C.c_void_p()
        _lib.event_create(C.byref(e0)); _lib.event_create(C.byref(e1))
        barrier()
        _lib.event_record(e0, stream())
        h0 = time.perf_counter()
        window[0] = h0
        for _ in range(steps):
            fn()
        if after is not None:
            after()
        _lib.event_record(e1, stream())
        host_ms[0] = (time.perf_counter() - h0) * 1e3 / steps    # time the host needs to queue one step
        _lib.event_sync(e1)
        window[1] = time.perf_counter()
        barrier()
        ms = C.c_float()
        _lib.event_elapsed_ms(e0, e1, C.byref(ms))
        t = DeviceArray.from_numpy(np.array([ms.value], np.float32))
        if acc.comm is not None:
            acc.comm.all_reduce(t, t, op="max")
        return float(t.numpy()[0])

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()      # before the warm-up: nvidia-smi needs a few hundred ms to deliver its first sample
    for _ in range(max(args.warmup, 3)):
        step_resident()
    if acc.comm is not None:
        _lib.device_sync()
        acc.comm.exposed_ms()                      # drop the warm-up's records
    launches0 = _lib.launch_count()
    ms_total = timed(step_resident, args.steps)
    launches = _lib.launch_count() - launches0
    # Host time to queue ONE step into an empty stream. (Averaged over the K timed steps the host
    # figure includes the time it is blocked on a full launch queue, two to three steps ahead of
    # the device.)
    _lib.device_sync()
    h0 = time.perf_counter()
    step_resident()
    host_queue_ms = (time.perf_counter() - h0) * 1e3
    _lib.device_sync()
    exposed = acc.comm.exposed_ms() if acc.comm is not None else None
    clocks = sampler.summary(tuple(window)) if rank == 0 else None
    # The roofline of the dominant kernel comes from a second pass over the same K steps with a
    # CUDA event on either side of every GEMM launch; the event records cost the step 2-5 %, so
    # they stay out of the pass that `value` is taken from. A third pass does the same for the
    # attention kernels.
    _lib.prof_begin(1)
    ms_prof = timed(step_resident, args.steps)
    gemm_ms, gemm_n, gemm_flops = C.c_double(), C.c_int64(), C.c_double()
    _lib.prof_end(C.byref(gemm_ms), C.byref(gemm_n), C.byref(gemm_flops))
    _lib.prof_begin(2)
    ms_prof2 = timed(step_resident, args.steps)
    attn_ms, attn_n, attn_flops = C.c_double(), C.c_int64(), C.c_double()
    _lib.prof_end(C.byref(attn_ms), C.byref(attn_n), C.byref(attn_flops))
    for _ in range(2):
        step_e2e()
    e2e_drain()
    ms_e2e = timed(step_e2e, args.steps, after=e2e_drain)
    final_loss = e2e_state["last"]
    flag = C.c_int(0)
    _lib.device_flag_read(C.byref(flag), stream())
    free_b, total_b = C.c_size_t(), C.c_size_t()
    _lib.mem_info(C.byref(free_b), C.byref(total_b))

    # Replicas must have stayed identical: the loss of one batch that every rank evaluates (rank
    # 0's first batch, generated again here) and the sum of the fp32 master weights, max - min
    # over ranks.
    agreement = None
    if acc.comm is not None:
        common = np.random.default_rng(100).integers(0, vocab_data, (micro_b, ctx + 1))
        cx = DeviceArray.from_numpy(common[:, :-1].astype(np.int32))
        cy = DeviceArray.from_numpy(common[:, 1:].astype(np.int32))
        with no_grad():
            ev_loss = forward_loss(cx, cy)
        pair = DeviceArray.zeros((4,), "float32")
        _lib.memcpy_d2d(pair.ptr, ev_loss.data.ptr, 4, stream())
        master = acc._flat.master
        _lib.sum_f32(master.ptr, _lib.F32, master.size, pair.ptr + 4, stream())
        h = pair.numpy()
        both = DeviceArray.from_numpy(np.array([h[0], h[1], -h[0], -h[1]], np.float32))
        acc.comm.all_reduce(both, both, op="max")
        b = both.numpy()
        agreement = {"eval_loss": float(h[0]), "eval_loss_spread": float(b[0] + b[2]),
                     "master_weight_sum": float(h[1]), "master_weight_sum_spread": float(b[1] + b[3])}

    # N = 1 only, outside `value`: a longer run at the accumulation the 8-GPU configuration uses
    # per rank, so that the scaling curve has a sustained, accumulation-matched single-GPU figure.
    sustained = None
    if world == 1 and args.sustained_seconds > 0:
        acc.gradient_accumulation_steps = 4
        acc.scaler.accum_steps = 4
        acc.step_counter = 0
        acc.scaler.update(None)                   # refreshes 1 / (scale * accumulation) on the device
        per_step_ms = 4 * ms_total / args.steps
        n_sus = max(3, int(np.ceil(args.sustained_seconds * 1e3 / per_step_ms)))
        step_resident()
        ms_sus = timed(step_resident, n_sus)
        sustained = {"grad_accum": 4, "steps": n_sus, "seconds": ms_sus / 1e3,
                     "ms_per_micro_batch": ms_sus / n_sus / 4,
                     "tokens_per_s": micro_b * ctx * 4 * n_sus / (ms_sus / 1e3),
                     "clocks": sampler.summary(tuple(window)) if rank == 0 else None}
    if rank == 0:
        sampler.stop()

    if rank == 0:
        tokens_per_step = micro_b * ctx * accum * world
        ms_step = ms_total / args.steps
        value = tokens_per_step / (ms_step / 1e3)
        e2e_val = tokens_per_step / (ms_e2e / args.steps / 1e3)
        peaks = measured_peaks()
        ftok = flops_per_token(w["cfg"], ctx)
        achieved = gemm_flops.value / (gemm_ms.value / 1e3) / 1e12 if gemm_ms.value > 0 else None
        cap = gemm_capture()
        out = {
            "metric": w["metric"], "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": config_dict(world, accum, args.config),
            "mfu": value / world * ftok / 2.25e15, "mfu_of_measured_peak": value / world * ftok / (peaks["tflops"] * 1e12),
            "flops_per_token": ftok,
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": 2 * nbytes * accum,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches), "host_queue_ms_per_step": host_queue_ms,
            "roofline": {"kernel": "gemm_tc_kernel (tcgen05 GEMM, all launches of the timed region)", "bound": "tensor",
                         "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": (achieved / peaks["tflops"]) if achieved else None, "peak_source": peaks["source"],
                         "launches": int(gemm_n.value), "ms_per_launch": gemm_ms.value / max(1, gemm_n.value),
                         "share_of_step": gemm_ms.value / ms_prof,
                         "measured_in": "second pass of the same steps with CUDA events around every GEMM launch",
                         "traffic": cap.get("traffic_bytes_per_launch"),
                         "traffic_unit": "bytes per launch, " + str(cap.get("workload", "no capture on file")),
                         "traffic_source": cap.get("summary"),
                         "library_same_data_tflops": cap.get("library_same_data_tflops")},
            "attention": {"achieved_tflops": attn_flops.value / (attn_ms.value / 1e3) / 1e12 if attn_ms.value > 0 else None,
                          "launches": int(attn_n.value), "ms_per_step": attn_ms.value / args.steps,
                          "share_of_step": attn_ms.value / ms_prof2,
                          "measured_in": "third pass, CUDA events around every attention launch (forward and backward)"},
            "memory": {"device_used_gb": (total_b.value - free_b.value) / 1e9, "device_total_gb": total_b.value / 1e9},
            "clocks": clocks, "final_loss": final_loss, "device_flag": flag.value,
        }
        if args.config == "d20":
            out["config"]["loss_mode"] = args.loss_mode
        if exposed is not None:
            out["comm"] = {"exposed_ms_per_optimizer_step": exposed,
                           "note": "time the compute stream waited for the last gradient buckets, rank 0"}
        if agreement is not None:
            out["rank_agreement"] = agreement
        if sustained is not None:
            out["sustained"] = sustained
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline_sample(args.config)
        print(json.dumps(out))
    if acc.comm is not None:
        acc.end_training()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--config", default="gpt2", choices=sorted(WORKLOADS))
    ap.add_argument("--loss-mode", default="fused", choices=["logits", "fused", "chunked"],
                    help="d20 only: how the model's forward produces the loss (see nanochat_gpt.GPT.loss_mode)")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="N = 1: length of the extra accumulation-4 run reported under `sustained` (0 = skip)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gemm-tile-policy", type=int, default=0, choices=[0, 1, 2],
                    help="0 automatic (default), 1 single-CTA GEMM tiles only, 2 CTA pairs; for A/B runs")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_own(args)


if __name__ == "__main__":
    main()
