"""Small stand-alone cases of each hot kernel, sized for a profiler capture:
inputs larger than the 126 MB L2 where DRAM figures matter, under 2 GB held on
the device, a handful of launches.

    python kernel_cases.py {gemm|attn|attn128|mem|adamw|gemm_vs_library|gemm_shapes|power|suite}

gemm : the GPT-2 124M qkv projection of one 16x1024-token micro-batch
       (16384x768 @ 768x2304, fp16), five launches
attn : causal flash attention forward + backward, 4x12x1024x64 fp16, three rounds
attn128 : the same at head_dim 128, 16x10x2048x128 fp16 (half a nanochat-d20 micro-batch: 160
       heads, enough for the head-grouped tile order to matter), two rounds
mem  : LayerNorm forward/backward (16384x768), cross entropy forward/backward
       (4096x50304), GELU backward (16384x3072), softmax (16384x1024), three rounds
adamw: fused AdamW over one 64M-element fp32 tensor, three steps
gemm_vs_library : the lm_head GEMM (16384x50304x768, fp16) timed for 300 back-to-back launches
       with CUDA events, this library's kernel and torch.matmul (cuBLAS) side by side, on
       random-normal, small-integer and all-zero operands. Throughput on a power-capped B200
       depends on the operand values (bit toggling), so a roofline fraction only means
       something against a library number taken on the same data.
gemm_shapes : every GEMM of one GPT-2 124M micro-batch (16384 tokens: qkv, out-proj, fc1, fc2, lm_head;
       forward, dgrad, wgrad, with the epilogues the model uses) timed back to back on random-normal
       data, this library's kernel next to torch.matmul (cuBLAS) on the same operands.
power : board power (nvidia-smi, 20 ms samples) while one kernel at a time loops for ~1.5 s at the
       GPT-2 124M shapes: time per launch x median power = energy per launch. On a 1 kW board the
       training step runs at the power cap, so its floor is the sum of these energies / 1 kW.
suite : the isolated fused-op suite at its stated shapes (attention 8x12x1024x64 causal, LayerNorm
       16384x768, softmax 16384x1024, cross entropy 8192x50304, matmul 8192x768x3072), each op
       forward and backward in fp16 and fp32, timed with CUDA events over inputs that rotate
       through more than the 126 MB L2, with the achieved TFLOP/s or GB/s and its fraction of the
       measured peak (MEASURED_PEAKS.json beside this file, else 6650 GB/s / 1590 TFLOP/s).
"""
import json
import os
import sys

import numpy as np

from mytorch_b200 import fused_ops as F
from mytorch_b200.array import DeviceArray, synchronize

ROWS = 16384


def main(which):
    r = np.random.default_rng(0)

    def randn(shape, dt="float16"):
        return DeviceArray.from_numpy(r.standard_normal(shape).astype(np.float32), dt)

    if which == "gemm":
        a, b = randn((ROWS, 768)), randn((2304, 768))
        out = DeviceArray.empty((ROWS, 2304), "float16")
        for _ in range(5):
            F.gemm(a, b, trans_b=True, out=out)
    elif which == "attn":
        q, k, v, do = (randn((4, 12, 1024, 64)) for _ in range(4))
        for _ in range(3):
            _, _, _, o, m = F.fused_sdpa_forward(q, k, v, causal=True)
            F.fused_sdpa_backward(do, q, k, v, o, m, causal=True)
    elif which == "attn128":
        q, k, v, do = (randn((16, 10, 2048, 128)) for _ in range(4))
        for _ in range(2):
            _, _, _, o, m = F.fused_sdpa_forward(q, k, v, causal=True)
            F.fused_sdpa_backward(do, q, k, v, o, m, causal=True)
    elif which == "mem":
        x, g, dy = randn((ROWS, 768)), randn((768,)), randn((ROWS, 768))
        lg = randn((4096, 50304))
        lab = DeviceArray.from_numpy(r.integers(0, 50257, 4096).astype(np.int32))
        u, du = randn((ROWS, 3072)), randn((ROWS, 3072))
        for _ in range(3):
            y, mu, rs = F.fused_layernorm_forward(x, g, None)
            F.fused_layernorm_backward(x, mu, rs, dy, g, None)
            loss, lse = F.fused_cross_entropy_forward(lg, lab)
            F.fused_cross_entropy_backward(lg, lab, lse, scale=1.0)
            F.fused_cross_entropy_forward_backward(lg, lab)      # what the training step runs
            F.fused_activation_backward(u, du, "gelu")
            F.fused_softmax_forward(randn((ROWS, 1024)))
    elif which == "adamw":
        import mytorch_b200 as mt
        n = 64 * 1024 * 1024
        p = mt.Tensor(DeviceArray.zeros((n,), "float32"), requires_grad=True)
        p.is_param = True
        opt = mt.optim.AdamW([{"params": [p], "weight_decay": 0.1}], lr=1e-3)
        for _ in range(3):
            p.grad = DeviceArray.zeros((n,), "float32")
            opt.step()
    elif which == "gemm_vs_library":
        gemm_vs_library(r)
        return
    elif which == "gemm_shapes":
        gemm_shapes(r)
        return
    elif which == "power":
        power_by_kernel(randn, r)
        return
    elif which == "suite":
        op_suite(r)
        return
    else:
        raise SystemExit(__doc__)
    synchronize()
    print("done", which)


def op_suite(r):
    """Times every op of the isolated suite, forward and backward, fp16 and fp32."""
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as fh:
            pk = json.load(fh)
        hbm, tf, src = pk["hbm_gbs"], pk["bf16_tflops"], "of measured"
    except Exception:
        hbm, tf, src = 6650.0, 1590.0, "of fallback"
    print(f"peaks: HBM {hbm:.0f} GB/s, tensor {tf:.0f} TFLOP/s (burst) - fractions are {src}")
    print(f"{'op':34s} {'dtype':8s} {'us':>9s} {'achieved':>16s} {'frac':>6s}")

    def report(name, dt, ms, flops=None, nbytes=None):
        if flops is not None:
            a = flops / ms / 1e9
            # fp32 GEMM and attention run on the CUDA cores (full fp32 for the 1e-4 parity bar): no tensor roofline
            frac = f"{a / tf:6.3f}" if dt == "float16" else "   n/a"
            print(f"{name:34s} {dt:8s} {ms * 1e3:9.1f} {a:10.1f} TFLOP/s {frac}", flush=True)
        else:
            a = nbytes / ms / 1e6
            print(f"{name:34s} {dt:8s} {ms * 1e3:9.1f} {a:10.0f} GB/s    {a / hbm:6.3f}", flush=True)

    def rotating(make, min_bytes=300e6):
        """Enough independent input sets that consecutive launches never find their data in L2."""
        first = make()
        per = sum(a.nbytes for a in first if isinstance(a, DeviceArray))
        sets = [first] + [make() for _ in range(max(1, int(min_bytes / max(per, 1))))]
        return sets

    def timed(sets, fn, iters=None):
        n = len(sets)
        it = [0]

        def one():
            fn(*sets[it[0] % n])
            it[0] += 1
        per = _time_own(one, 3, warm=2)
        n_it = iters or max(10, min(200, int(300.0 / max(per, 1e-3))))
        return _time_own(one, n_it, host_us_per_call=60.0 if per < 0.2 else 0.0)

    for dt in ("float16", "float32"):
        sz = 2 if dt == "float16" else 4
        rn = lambda shape: DeviceArray.from_numpy(r.standard_normal(shape, dtype=np.float32), dt)
        # (a) attention
        B, H, S, D = 8, 12, 1024, 64
        sets = rotating(lambda: tuple(rn((B, H, S, D)) for _ in range(4)))
        iters = 50 if dt == "float16" else 5
        ms = timed(sets, lambda q, k, v, do: F.fused_sdpa_forward(q, k, v, causal=True), iters)
        report("attention fwd 8x12x1024x64 causal", dt, ms, flops=2.0 * B * H * S * S * D)
        saved = [F.fused_sdpa_forward(q, k, v, causal=True)[3:] for q, k, v, _ in sets]
        full = [s_ + tuple(o) for s_, o in zip(sets, saved)]
        ms = timed(full, lambda q, k, v, do, o, m: F.fused_sdpa_backward(do, q, k, v, o, m, causal=True), iters)
        report("attention bwd", dt, ms, flops=5.0 * B * H * S * S * D)
        del sets, saved, full
        # (b) LayerNorm
        N, E = 16384, 768
        g, b = DeviceArray.from_numpy(np.ones(E, np.float32), dt), DeviceArray.from_numpy(np.zeros(E, np.float32), dt)
        sets = rotating(lambda: (rn((N, E)), rn((N, E))))
        ms = timed(sets, lambda x, dy: F.fused_layernorm_forward(x, g, b))
        report("layernorm fwd 16384x768", dt, ms, nbytes=2.0 * N * E * sz)
        full = [(x, dy) + tuple(F.fused_layernorm_forward(x, g, b)[1:]) for x, dy in sets]
        ms = timed(full, lambda x, dy, mu, rs: F.fused_layernorm_backward(x, mu, rs, dy, g, b))
        report("layernorm bwd", dt, ms, nbytes=3.0 * N * E * sz)
        del sets, full
        # (c) softmax
        N, Cc = 16384, 1024
        sets = rotating(lambda: (rn((N, Cc)), rn((N, Cc))))
        ms = timed(sets, lambda x, dy: F.fused_softmax_forward(x))
        report("softmax fwd 16384x1024", dt, ms, nbytes=2.0 * N * Cc * sz)
        full = [(F.fused_softmax_forward(x), dy) for x, dy in sets]
        ms = timed(full, lambda s_, dy: F.fused_softmax_backward(dy, s_))
        report("softmax bwd", dt, ms, nbytes=3.0 * N * Cc * sz)
        del sets, full
        # (d) cross entropy: one set is already 0.8-1.6 GB
        N, Cc = 8192, 50304
        lab = DeviceArray.from_numpy(r.integers(0, 50257, N).astype(np.int32))
        x = rn((N, Cc))
        ms = _time_own(lambda: F.fused_cross_entropy_forward(x, lab), 20)
        report("cross entropy fwd 8192x50304", dt, ms, nbytes=1.0 * N * Cc * sz)
        _, lse = F.fused_cross_entropy_forward(x, lab)
        ms = _time_own(lambda: F.fused_cross_entropy_backward(x, lab, lse, scale=1.0), 20)   # in place: values stay bounded
        report("cross entropy bwd (in place)", dt, ms, nbytes=2.0 * N * Cc * sz)
        ms = _time_own(lambda: F.fused_cross_entropy_forward_backward(x, lab, scale=float(N)), 20)
        report("cross entropy fwd+grad, one pass", dt, ms, nbytes=2.0 * N * Cc * sz)
        del x
        # (e) matmul as Linear: X[8192,768], W[3072,768]
        M, Kk, Nn = 8192, 768, 3072
        sets = rotating(lambda: (rn((M, Kk)), rn((Nn, Kk)), rn((M, Nn))))
        iters = 100 if dt == "float16" else 5
        ms = timed(sets, lambda x, w, dy: F.gemm(x, w, trans_b=True), iters)
        report("matmul fwd 8192x768x3072", dt, ms, flops=2.0 * M * Kk * Nn)
        ms = timed(sets, lambda x, w, dy: F.gemm(dy, w), iters)
        report("matmul dgrad", dt, ms, flops=2.0 * M * Kk * Nn)
        ms = timed(sets, lambda x, w, dy: F.gemm(dy, x, trans_a=True, out_dtype="float32"), iters)
        report("matmul wgrad (fp32 out)", dt, ms, flops=2.0 * M * Kk * Nn)
        del sets


_BLOCKER = []


def _time_own(fn, iters, warm=3, host_us_per_call=0.0):
    """Mean device time of `fn` over `iters` back-to-back calls (CUDA events on the compute
    stream). A call costs the host 20-50 us of Python and ctypes; for kernels shorter than that
    the device would idle between launches and the events would time the host. With
    host_us_per_call > 0 the stream is first kept busy with large memsets for about that long per
    call, so that every timed launch is already queued when the first one starts."""
    import ctypes as C
    from mytorch_b200 import _lib
    from mytorch_b200.array import stream
    for _ in range(warm):
        fn()
    e0, e1 = C.c_void_p(), C.c_void_p()
    _lib.event_create(C.byref(e0)); _lib.event_create(C.byref(e1))
    if host_us_per_call > 0:
        if not _BLOCKER:
            _BLOCKER.append(DeviceArray.empty((2 << 30,), "uint8"))
        for _ in range(int(iters * host_us_per_call / 300.0) + 1):      # one 2 GB memset takes ~0.3 ms
            _lib.memset(_BLOCKER[0].ptr, 0, _BLOCKER[0].nbytes, stream())
    _lib.event_record(e0, stream())
    for _ in range(iters):
        fn()
    _lib.event_record(e1, stream())
    _lib.event_sync(e1)
    ms = C.c_float()
    _lib.event_elapsed_ms(e0, e1, C.byref(ms))
    return ms.value / iters


def power_by_kernel(randn, r, seconds=1.5):
    import subprocess, threading, time
    import mytorch_b200 as mt
    samples = []

    def sampler(stop):
        p = subprocess.Popen(["nvidia-smi", "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits",
                              "-lms", "20"], stdout=subprocess.PIPE, text=True)
        while not stop.is_set():
            line = p.stdout.readline()
            if "," in line:
                samples.append([float(c) for c in line.split(",")])
        p.terminate()      # the exact child started above

    def sampled(body):
        samples.clear()
        stop = threading.Event()
        th = threading.Thread(target=sampler, args=(stop,))
        th.start()
        time.sleep(0.05)
        out = body()
        stop.set()
        th.join()
        tail = samples[len(samples) // 3:] or [[0.0, 0.0]]     # skip the ramp
        return out, float(np.median([s[0] for s in tail])), float(np.median([s[1] for s in tail]))

    _, clk, watts = sampled(lambda: time.sleep(1.0))
    print(f"{'idle (context up)':28s}: {'':10s}   clock {clk:5.0f} MHz | {watts:5.0f} W", flush=True)

    def run(name, fn):
        per = _time_own(fn, 10)
        iters = max(10, int(seconds * 1e3 / per))
        ms, clk, watts = sampled(lambda: _time_own(fn, iters))
        print(f"{name:28s}: {ms * 1e3:8.1f} us | clock {clk:5.0f} MHz | {watts:5.0f} W | {ms * watts:7.2f} mJ per launch",
              flush=True)

    a, b = randn((ROWS, 768)), randn((2304, 768))
    out = DeviceArray.empty((ROWS, 2304), "float16")
    run("gemm 16384x2304x768", lambda: F.gemm(a, b, trans_b=True, out=out))
    q, k, v, do = (randn((16, 12, 1024, 64)) for _ in range(4))
    _, _, _, o, m = F.fused_sdpa_forward(q, k, v, causal=True)
    run("attention fwd 16x12x1024x64", lambda: F.fused_sdpa_forward(q, k, v, causal=True))
    run("attention bwd", lambda: F.fused_sdpa_backward(do, q, k, v, o, m, causal=True))
    x, g, dy = randn((ROWS, 768)), randn((768,)), randn((ROWS, 768))
    y, mu, rs = F.fused_layernorm_forward(x, g, None)
    run("layernorm fwd 16384x768", lambda: F.fused_layernorm_forward(x, g, None))
    run("layernorm bwd", lambda: F.fused_layernorm_backward(x, mu, rs, dy, g, None))
    lg = randn((ROWS, 50304))
    lab = DeviceArray.from_numpy(r.integers(0, 50257, ROWS).astype(np.int32))
    run("cross entropy fwd+grad", lambda: F.fused_cross_entropy_forward_backward(lg, lab))
    n = 124 * 1024 * 1024
    p = mt.Tensor(DeviceArray.zeros((n,), "float32"), requires_grad=True)
    p.is_param = True
    opt = mt.optim.AdamW([{"params": [p], "weight_decay": 0.1}], lr=1e-3)
    gz = DeviceArray.zeros((n,), "float32")

    def step():
        p.grad = gz
        opt.step()
    run("AdamW step, 130M fp32", step)


def gemm_shapes(r, M=16384, iters=100):
    """One line per GEMM of the GPT-2 124M step: this library (with the epilogue the model uses)
    and torch.matmul on the same random-normal operands, microseconds and TFLOP/s."""
    import torch
    d, V = 768, 50304

    def rn(shape, dt="float16"):
        return DeviceArray.from_numpy(r.standard_normal(shape, dtype=np.float32), dt)

    def tt(a):
        return torch.from_numpy(a.numpy()).cuda()

    def time_torch(fn):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    print(f"{'GEMM (M=16384 tokens)':44s} {'N':>6s} {'K':>6s} | {'this library':>22s} | {'torch.matmul':>22s} | ratio")
    total_own = total_lib = 0.0
    for name, n_out, k_in, count in (("qkv", 3 * d, d, 12), ("out-proj", d, d, 12), ("fc1", 4 * d, d, 12),
                                     ("fc2", d, 4 * d, 12), ("lm_head", V, d, 1)):
        x, w, dy = rn((M, k_in)), rn((n_out, k_in)), rn((M, n_out))
        res, aux = rn((M, n_out)), rn((M, k_in))
        tx, tw, tdy = tt(x), tt(w), tt(dy)
        y = DeviceArray.empty((M, n_out), "float16")
        dx = DeviceArray.empty((M, k_in), "float16")
        dw = DeviceArray.zeros((n_out, k_in), "float32")
        variants = []
        if name == "fc1":
            variants.append(("fwd + GELU, derivative stored", lambda: F.gemm(x, w, trans_b=True, act="gelu", preact="grad"), M, n_out, k_in))
        elif name in ("out-proj", "fc2"):
            variants.append(("fwd + residual add", lambda: F.gemm(x, w, trans_b=True, out=y, aux=res, aux_mode=1), M, n_out, k_in))
        else:
            variants.append(("fwd", lambda: F.gemm(x, w, trans_b=True, out=y), M, n_out, k_in))
        if name == "fc2":
            variants.append(("dgrad * act'(.)", lambda: F.gemm(dy, w, out=dx, aux=aux, aux_mode=5), M, k_in, n_out))
        else:
            variants.append(("dgrad", lambda: F.gemm(dy, w, out=dx), M, k_in, n_out))
        variants.append(("wgrad (fp32, split-K add)", lambda: F.gemm(dy, x, trans_a=True, out=dw, accumulate=2), n_out, k_in, M))
        libs = [lambda: torch.matmul(tx, tw.t()), lambda: torch.matmul(tdy, tw), lambda: torch.matmul(tdy.t(), tx)]
        for (label, fn, mm, nn, kk), lib in zip(variants, libs):
            own = _time_own(fn, iters)
            ref = time_torch(lib)
            fl = 2.0 * mm * nn * kk
            total_own += own * count
            total_lib += ref * count
            print(f"{name + ' ' + label:44s} {nn:6d} {kk:6d} | {own * 1e3:8.1f} us {fl / own / 1e9:6.0f} TF/s | "
                  f"{ref * 1e3:8.1f} us {fl / ref / 1e9:6.0f} TF/s | {ref / own:5.2f}", flush=True)
        del x, w, dy, res, aux, tx, tw, tdy, y, dx, dw
    print(f"sum over one micro-batch (12 layers + head): this library {total_own:.2f} ms, torch.matmul {total_lib:.2f} ms "
          "(the library side carries the fused epilogues; the torch side is the bare product)")


def gemm_vs_library(r, m=16384, n=50304, k=768, iters=300):
    import ctypes as C
    import torch
    from mytorch_b200 import _lib
    from mytorch_b200.array import stream

    def time_own(fn):
        for _ in range(3):
            fn()
        e0, e1 = C.c_void_p(), C.c_void_p()
        _lib.event_create(C.byref(e0)); _lib.event_create(C.byref(e1))
        _lib.event_record(e0, stream())
        for _ in range(iters):
            fn()
        _lib.event_record(e1, stream())
        _lib.event_sync(e1)
        ms = C.c_float()
        _lib.event_elapsed_ms(e0, e1, C.byref(ms))
        return ms.value / iters

    def time_torch(fn):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    flop = 2.0 * m * n * k
    for dist in ("randn", "small_ints", "zeros"):
        if dist == "randn":
            a, b = r.standard_normal((m, k)), r.standard_normal((n, k))
        elif dist == "small_ints":
            a, b = r.integers(-2, 3, (m, k)), r.integers(-2, 3, (n, k))
        else:
            a, b = np.zeros((m, k)), np.zeros((n, k))
        a, b = a.astype(np.float32), b.astype(np.float32)
        A, B = DeviceArray.from_numpy(a, "float16"), DeviceArray.from_numpy(b, "float16")
        out = DeviceArray.empty((m, n), "float16")
        own = time_own(lambda: F.gemm(A, B, trans_b=True, out=out))
        ta, tb = torch.from_numpy(a).cuda().half(), torch.from_numpy(b).cuda().half()
        to = torch.empty((m, n), device="cuda", dtype=torch.float16)
        lib = time_torch(lambda: torch.matmul(ta, tb.t(), out=to))
        print(f"{dist:10s}: this library {own * 1e3:7.1f} us {flop / own / 1e9:5.0f} TFLOP/s | "
              f"torch.matmul {lib * 1e3:7.1f} us {flop / lib / 1e9:5.0f} TFLOP/s", flush=True)
        del ta, tb, to


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "")
