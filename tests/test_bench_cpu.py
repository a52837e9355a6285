"""Host-side logic of bench.py that needs no GPU."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def row(t, mhz, watts, cap="Not Active"):
    return [t, "0", str(mhz), "1965", str(watts), "0x4", "Not Active", "Not Active", "Not Active", cap]


def test_clock_samples_are_taken_from_the_timed_window():
    b = load_bench()
    s = b.ClockSampler(0)
    s.rows = [row(0.5, 120, 200.0), row(1.1, 1700, 900.0, "Active"), row(1.2, 1750, 950.0, "Active"),
              row(1.3, 1800, 940.0, "Active"), row(2.5, 1965, 300.0)]
    got = s.stop((1.0, 2.0))
    assert got["samples"] == 3 and got["sm_mhz"] == 1750.0 and got["sm_max_mhz"] == 1965.0
    assert got["power_w"] == 940.0 and got["reasons"] == ["sw_power_cap"]
    # no sample inside the window: every sample counts, and an idle clock shows as such
    got = s.stop((3.0, 4.0))
    assert got["samples"] == 5 and got["sm_mhz"] == 1750.0
    assert b.ClockSampler(0).stop((0.0, 1.0))["samples"] == 0


def test_accumulation_keeps_the_global_batch():
    b = load_bench()
    assert b.accum_for(1) == 1
    for n in (2, 4, 8):
        cfg = b.config_dict(n, b.accum_for(n))
        assert cfg["global_batch_tokens"] == 524288 and cfg["grad_accum"] * n == 32


def test_d20_workload_arithmetic():
    b = load_bench()
    assert b.accum_for(1, "d20") == 1 and b.accum_for(8, "d20") == 1 and b.accum_for(2, "d20") == 4
    for n in (2, 4, 8):
        assert b.config_dict(n, b.accum_for(n, "d20"), "d20")["global_batch_tokens"] == 524288
    # 6 * P_mm + 6 * L * T * d with P_mm = 477 102 080 matmul weights (untied head, no embedding)
    assert b.flops_per_token(b.D20_CFG, 2048) == 6 * 477102080 + 6 * 20 * 2048 * 1280
    assert b.flops_per_token() == 798031872


def test_roofline_traffic_comes_from_the_capture_on_file():
    b = load_bench()
    cap = b.gemm_capture()
    assert cap["traffic_bytes_per_launch"] == cap["dram_bytes_read"] + cap["dram_bytes_write"]
    assert os.path.exists(os.path.join(ROOT, cap["summary"])) and os.path.exists(os.path.join(ROOT, cap["library_summary"]))
