"""Benchmark of the GPT-2 124M training step (tokens/s and MFU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Own arm: one process per GPU (torchrun-style env for N > 1). A step is one
optimizer step: forward + backward of `accum` micro-batches of 16 x 1024 tokens,
gradient all-reduce (N > 1), global-norm clip, fused AdamW with fp16 dynamic
loss scaling. N = 1 runs the single-GPU configuration (accum = 1); N > 1 the
data-parallel one (global batch 524288 tokens, accum = 32 / N). Timing: CUDA
events on the compute stream around exactly K steps, bracketed by barrier +
synchronize, max over ranks. `value` has the token ids resident in HBM; `e2e`
repeats the K steps with host batches (pinned -> device copy of ids and labels
and a device -> host read of the loss inside every step).

Reference arm (`--impl reference`): the reference's algorithm for the same step
on the host cores (the NumPy oracle, which is pinned to the reference by the
golden vectors), on a bounded sample of the workload: the full 124M model,
one sequence of 1024 tokens per step.
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


def flops_per_token(cfg=CFG, ctx=CTX):
    """fwd+bwd model FLOPs per token, causal-exact attention: 6*P_mm + 6*L*T*d."""
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

    def stop(self, window=None):
        """Summary of the samples taken inside `window` = (t0, t1) in perf_counter seconds (all
        samples when none fell inside it)."""
        if self.proc is not None:
            self.proc.terminate()      # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = self.rows
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


# --------------------------------------------------------------- reference arm ----
def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    from oracle import gpt2 as og
    cores = os.cpu_count() or 1
    cfg = og.GPT2Config(**CFG)
    params = og.init_params(cfg, seed=0)
    opt = og.AdamW(params, LR, 0.9, 0.95, 1e-8, WD)
    rng = np.random.default_rng(0)
    times = []
    for i in range(args.warmup + args.steps):
        x, y = og.synthetic_batch(rng, 1, CTX, VOCAB_DATA)
        t0 = time.perf_counter()
        loss, _, cache = og.forward(params, cfg, x, y)
        grads = og.backward(params, cfg, cache)
        from oracle import ops as O
        O.clip_grad_norm(list(grads.values()), CLIP)
        opt.step(params, grads)
        dt = time.perf_counter() - t0
        if i >= args.warmup:
            times.append(dt)
    sec = float(np.mean(times))
    val = CTX / sec
    sample = "full 124M model, 1 sequence x 1024 tokens per step (of 16 x 1024), fp32 NumPy"
    print(json.dumps({
        "impl": "reference", "metric": "GPT-2 124M train tokens/s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.gpus, accum_for(args.gpus)),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_baseline_sample(seconds_budget=30.0):
    """The oracle's step on a bounded sample (1 x 1024 tokens, full model), one
    timed step after one warm-up, or just the warm-up if that already took long."""
    from oracle import gpt2 as og
    from oracle import ops as O
    cfg = og.GPT2Config(**CFG)
    params = og.init_params(cfg, seed=0)
    opt = og.AdamW(params, LR, 0.9, 0.95, 1e-8, WD)
    rng = np.random.default_rng(0)
    times = []
    for i in range(2):
        x, y = og.synthetic_batch(rng, 1, CTX, VOCAB_DATA)
        t0 = time.perf_counter()
        loss, _, cache = og.forward(params, cfg, x, y)
        grads = og.backward(params, cfg, cache)
        O.clip_grad_norm(list(grads.values()), CLIP)
        opt.step(params, grads)
        times.append(time.perf_counter() - t0)
        if times[-1] > seconds_budget / 2:
            break
    sec = times[-1]
    return {"value": CTX / sec, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": "full 124M model, 1 sequence x 1024 tokens (of 16 x 1024) per step, fp32 NumPy oracle, "
                      f"{len(times)} step(s), last timed"}


def accum_for(n_gpus):
    return 1 if n_gpus == 1 else max(1, GLOBAL_TOKENS // (MICRO_B * CTX * n_gpus))


def config_dict(n_gpus, accum):
    return {"workload": "GPT-2 124M (L12 H12 d768 ctx1024 vocab50304, tied) fp16 mixed precision, "
                        "AdamW lr6e-4 wd0.1 clip1.0, micro-batch 16x1024"
                        + ("" if n_gpus == 1 else f", DDP global batch {MICRO_B * CTX * n_gpus * accum} tokens"),
            "micro_batch": MICRO_B, "seq_len": CTX, "grad_accum": accum,
            "global_batch_tokens": MICRO_B * CTX * n_gpus * accum,
            "parallelism": f"dp{n_gpus}", "l2": "working set per step (>2 GB of activations, 1.6 GB logits) exceeds the 126 MB L2"}


# ------------------------------------------------------------------- own arm ----
def run_own(args):
    import mytorch_b200 as mt
    from mytorch_b200 import _lib
    from mytorch_b200.array import DeviceArray, stream
    from mytorch_b200.gpt2 import GPT2, GPT2Config

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")
    accum = accum_for(world)
    if args.gemm_tile_policy:
        _lib.gemm_tile_policy(args.gemm_tile_policy)
    acc = mt.Accelerator(num_gpus=world, rank=rank, gradient_accumulation_steps=accum, mixed_precision=True)
    np.random.seed(1234)                      # identical initial weights on every rank
    model = GPT2(GPT2Config(**CFG))
    decay, no_decay = [], []
    for _, p in model.named_parameters():
        (no_decay if len(p.shape) < 2 else decay).append(p)
    opt = mt.optim.AdamW([{"params": decay, "weight_decay": WD}, {"params": no_decay, "weight_decay": 0.0}],
                         lr=LR, beta1=0.9, beta2=0.95)
    model, opt = acc.prepare(model, opt)
    # the training loop never looks at the logits after the loss: let the loss overwrite them with
    # their gradient in its forward pass (one read + one write of the 1.65 GB instead of 2 + 1)
    loss_fn = mt.nn.CrossEntropyLoss(fused_backward=True)

    rng = np.random.default_rng(100 + rank)
    n_batches = 4
    host_ids = [rng.integers(0, VOCAB_DATA, (MICRO_B, CTX + 1)) for _ in range(n_batches)]
    dev_x = [DeviceArray.from_numpy(h[:, :-1].astype(np.int32)) for h in host_ids]
    dev_y = [DeviceArray.from_numpy(h[:, 1:].astype(np.int32)) for h in host_ids]

    # pinned host staging for the end-to-end pass
    nbytes = MICRO_B * CTX * 4
    pin = C.c_void_p()
    _lib.host_alloc(C.byref(pin), 2 * nbytes * n_batches + 64)
    pinned = np.ctypeslib.as_array((C.c_int32 * (2 * MICRO_B * CTX * n_batches)).from_address(pin.value))
    for i, h in enumerate(host_ids):
        pinned[(2 * i) * MICRO_B * CTX:(2 * i + 1) * MICRO_B * CTX] = h[:, :-1].reshape(-1)
        pinned[(2 * i + 1) * MICRO_B * CTX:(2 * i + 2) * MICRO_B * CTX] = h[:, 1:].reshape(-1)
    stage_x = DeviceArray.empty((MICRO_B, CTX), "int32")
    stage_y = DeviceArray.empty((MICRO_B, CTX), "int32")
    loss_pin = C.c_void_p()
    _lib.host_alloc(C.byref(loss_pin), 64)

    counter = [0]

    def micro(x, y):
        loss = loss_fn(model(mt.Tensor(x)), mt.Tensor(y))
        acc.backward(loss)
        acc.clip_grad_norm_(CLIP)
        opt.step()
        opt.zero_grad()
        return loss

    def step_resident():
        for _ in range(accum):
            i = counter[0] % n_batches
            counter[0] += 1
            loss = micro(dev_x[i], dev_y[i])
        return loss

    def step_e2e():
        for _ in range(accum):
            i = counter[0] % n_batches
            counter[0] += 1
            base = pin.value + (2 * i) * nbytes
            _lib.memcpy_h2d(stage_x.ptr, base, nbytes, stream())
            _lib.memcpy_h2d(stage_y.ptr, base + nbytes, nbytes, stream())
            loss = micro(stage_x, stage_y)
        _lib.memcpy_d2h(loss_pin.value, loss.data.ptr, 4, stream())
        _lib.stream_sync(stream())
        return loss

    def barrier():
        if acc.comm is not None:
            acc.comm.barrier()
        _lib.device_sync()

    host_ms = [0.0]
    window = [0.0, 0.0]      # host time of the last timed region, for the clock samples

    def timed(fn, steps):
        e0, e1 = C.c_void_p(), C.c_void_p()
        _lib.event_create(C.byref(e0)); _lib.event_create(C.byref(e1))
        barrier()
        _lib.event_record(e0, stream())
        h0 = time.perf_counter()
        window[0] = h0
        for _ in range(steps):
            fn()
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
    launches0 = _lib.launch_count()
    ms_total = timed(step_resident, args.steps)
    host_queue_ms = host_ms[0]
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop(tuple(window)) if rank == 0 else None
    # The roofline of the dominant kernel comes from a second pass over the same K steps with a
    # CUDA event on either side of every GEMM launch; the 2 x 147 event records per micro-batch
    # cost the step 2-3 %, so they stay out of the pass that `value` is taken from.
    _lib.prof_begin(1)
    ms_prof = timed(step_resident, args.steps)
    gemm_ms, gemm_n, gemm_flops = C.c_double(), C.c_int64(), C.c_double()
    _lib.prof_end(C.byref(gemm_ms), C.byref(gemm_n), C.byref(gemm_flops))
    final_loss = None
    for _ in range(2):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    final_loss = float(np.ctypeslib.as_array((C.c_float * 1).from_address(loss_pin.value))[0])
    flag = C.c_int(0)
    _lib.device_flag_read(C.byref(flag), stream())

    if rank == 0:
        tokens_per_step = MICRO_B * CTX * accum * world
        ms_step = ms_total / args.steps
        value = tokens_per_step / (ms_step / 1e3)
        e2e_val = tokens_per_step / (ms_e2e / args.steps / 1e3)
        peaks = measured_peaks()
        ftok = flops_per_token()
        achieved = gemm_flops.value / (gemm_ms.value / 1e3) / 1e12 if gemm_ms.value > 0 else None
        out = {
            "metric": "GPT-2 124M train tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": config_dict(world, accum),
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
                         # dram__bytes_read.sum + dram__bytes_write.sum of one captured launch of the
                         # qkv projection (16384x2304x768 fp16; profiles/gemm_tc_kernel_*.md): the
                         # operands are read once (30.3 MB), 26.4 MB of the 75.5 MB output reaches
                         # DRAM before the kernel ends, the rest stays in L2.
                         "traffic": 56.7e6, "traffic_unit": "bytes per launch (qkv projection, ncu)",
                         # torch.matmul (cuBLAS) on the lm_head shape with random-normal operands,
                         # same box type (profiles/gemm_vs_library_*.md): the same-data library figure
                         "library_same_data_tflops": 1136.0},
            "clocks": clocks, "final_loss": final_loss, "device_flag": flag.value,
        }
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline_sample()
        print(json.dumps(out))
    if acc.comm is not None:
        acc.end_training()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
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
