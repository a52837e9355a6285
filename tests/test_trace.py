"""The optional per-call tracing of the ctypes layer (environment variable MT_TRACE): NVTX ranges
and the CUDA-event timer. Both are chosen at import time, so every case runs in a child process."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_child(code, trace):
    env = dict(os.environ, PYTHONPATH=ROOT)
    env.pop("MT_TRACE", None)
    if trace is not None:
        env["MT_TRACE"] = trace
    return subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)


def test_tracing_is_off_by_default_and_rejects_unknown_modes():
    r = run_child("from mytorch_b200 import _lib\n"
                  "try:\n    _lib.trace_report()\nexcept RuntimeError as e:\n    print('off:', e)\n", None)
    assert r.returncode == 0 and "off: the per-call timer is off" in r.stdout, r.stderr
    r = run_child("import mytorch_b200", "everything")
    assert r.returncode != 0 and "expected 'nvtx' or 'time'" in r.stderr


def test_nvtx_ranges_wrap_compute_calls_only_and_pass_errors_through():
    code = ("from mytorch_b200 import _lib\n"
            "assert 'mt_gemm' in _lib.TRACED and 'mt_attn_bwd_gqa' in _lib.TRACED and 'mt_adamw_multi' in _lib.TRACED\n"
            "assert 'mt_malloc' not in _lib.TRACED and 'mt_event_record' not in _lib.TRACED\n"
            "_lib.range_push(b'outer'); _lib.range_pop()\n"          # no tool attached: both return at once
            "try:\n"
            "    _lib.layernorm_fwd(None, None, None, None, None, None, 4, 8, 1e-5, 0, None)\n"
            "except _lib.MTError as e:\n"
            "    print('error kept:', e)\n")
    r = run_child(code, "nvtx")
    assert r.returncode == 0, r.stderr
    assert "error kept:" in r.stdout and "bad arguments" in r.stdout


@pytest.mark.gpu
def test_event_timer_reports_calls_and_device_time_per_function():
    code = ("import numpy as np\n"
            "import mytorch_b200 as mt\n"
            "from mytorch_b200 import _lib, fused_ops as F\n"
            "from mytorch_b200.array import DeviceArray\n"
            "r = np.random.default_rng(0)\n"
            "x = DeviceArray.from_numpy(r.standard_normal((512, 768), dtype=np.float32), 'float16')\n"
            "g = DeviceArray.from_numpy(np.ones(768, np.float32), 'float16')\n"
            "for _ in range(5):\n"
            "    y, mu, rs = F.fused_layernorm_forward(x, g, None)\n"
            "for _ in range(3):\n"
            "    F.fused_layernorm_backward(x, mu, rs, y, g, None)\n"
            "rows = {n: (c, ms) for n, c, ms in _lib.trace_report(file=open('/dev/null', 'w'))}\n"
            "assert rows['mt_layernorm_fwd'][0] == 5 and rows['mt_layernorm_bwd'][0] == 3, rows\n"
            "assert all(ms > 0 for c, ms in rows.values()), rows\n"
            "ref = x.numpy().astype(np.float32)\n"
            "ref = (ref - ref.mean(1, keepdims=True)) / np.sqrt(ref.var(1, keepdims=True) + 1e-5)\n"
            "assert np.abs(y.numpy().astype(np.float32) - ref).max() < 2e-2\n"       # timed calls still compute
            "print('timed ok')\n")
    r = run_child(code, "time")
    assert r.returncode == 0 and "timed ok" in r.stdout, r.stderr[-2000:]
    assert "mt_layernorm_fwd" in r.stderr        # the report printed at interpreter exit
