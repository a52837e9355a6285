"""mt_layernorm_bwd_noalloc: the LayerNorm backward for callers that must not
allocate device memory while they run (all memory owned by the host program's
own arena, or a fixed, pre-audited budget). It keeps its reduction scratch in a
fixed array inside the library instead of taking it from the allocator.

Called through the C ABI twice in a row with different inputs and compared with
the allocating entry point mt_layernorm_bwd on the same inputs; the second call
checks that contents left in the shared scratch by the first do not leak into
the result. Every value of the `accumulate` bit mask is covered (1 = add into
dgamma/dbeta, 2 = add into dx), with the outputs pre-filled so that a dropped
or misplaced add shows. Tolerances are the ones of tests/test_ops_gpu.py (fp32
1e-4, fp16 1e-2 of the largest expected magnitude); the two entry points may
sum the per-block partials in a different grouping, so equality is not bitwise.
This file sorts last so that a run stopping at the first failure has already
executed every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(mt, entry, X, MU, RS, DY, G, rows, cols, dtype_code, accumulate, pre):
    from mytorch_b200.array import stream
    dx = mt.DeviceArray.from_numpy(pre[0], X.dtype)
    dg = mt.DeviceArray.from_numpy(pre[1], "float32")
    db = mt.DeviceArray.from_numpy(pre[2], "float32")
    entry(X.ptr, MU.ptr, RS.ptr, DY.ptr, G.ptr, dx.ptr, dg.ptr, db.ptr, rows, cols, accumulate, dtype_code, stream())
    return dx.numpy().astype(np.float64), dg.numpy().astype(np.float64), db.numpy().astype(np.float64)


@pytest.mark.parametrize("accumulate", [0, 1, 2, 3])
@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("float16", 1e-2)])
def test_noalloc_layernorm_backward_matches_allocating_entry_point(dtype, tol, accumulate):
    import mytorch_b200 as mt
    from mytorch_b200 import _lib, fused_ops as F
    code = {"float32": _lib.F32, "float16": _lib.F16}[dtype]
    r = np.random.default_rng(7)
    # the second call is smaller than the first, so stale partial rows of call 1 sit beyond its grid
    for rows, cols in [(2000, 512), (300, 256)]:      # within the fp32 limit of 512 columns
        x = r.standard_normal((rows, cols)).astype(np.float32)
        g = r.standard_normal(cols).astype(np.float32)
        dy = r.standard_normal((rows, cols)).astype(np.float32)
        pre = (r.standard_normal((rows, cols)).astype(np.float32), 10 * r.standard_normal(cols).astype(np.float32),
               10 * r.standard_normal(cols).astype(np.float32))
        X, G, DY = (mt.DeviceArray.from_numpy(a, dtype) for a in (x, g, dy))
        _, MU, RS = F.fused_layernorm_forward(X, G, None)
        want = _run(mt, _lib.layernorm_bwd, X, MU, RS, DY, G, rows, cols, code, accumulate, pre)
        got = _run(mt, _lib.layernorm_bwd_noalloc, X, MU, RS, DY, G, rows, cols, code, accumulate, pre)
        plain = _run(mt, _lib.layernorm_bwd, X, MU, RS, DY, G, rows, cols, code, 0, pre)
        for a, b, name in zip(got, want, ("dx", "dgamma", "dbeta")):
            scale = max(np.abs(b).max(), 1e-3)
            err = np.abs(a - b).max() / scale
            assert err <= tol, f"{name} {rows}x{cols} {dtype} accumulate={accumulate}: {err:.3e}"
        # the mask does what it says: the accumulating result is the plain result plus what was there
        if accumulate & 2:
            np.testing.assert_allclose(got[0], plain[0] + pre[0].astype(np.float16 if dtype == "float16" else np.float32),
                                       atol=(2e-2 if dtype == "float16" else 1e-4) * max(1.0, np.abs(plain[0]).max()))
        if accumulate & 1:
            np.testing.assert_allclose(got[1], plain[1] + pre[1], atol=tol * max(1.0, np.abs(plain[1]).max()))
            np.testing.assert_allclose(got[2], plain[2] + pre[2], atol=tol * max(1.0, np.abs(plain[2]).max()))


def test_noalloc_rejects_rows_wider_than_its_fixed_scratch():
    import mytorch_b200 as mt
    from mytorch_b200 import _lib
    from mytorch_b200.array import stream
    a = mt.DeviceArray.zeros((2, 4096), "float32")
    s = mt.DeviceArray.zeros((2,), "float32")
    with pytest.raises(_lib.MTError) as e:
        _lib.layernorm_bwd_noalloc(a.ptr, s.ptr, s.ptr, a.ptr, None, a.ptr, None, None, 2, 4096, 0, _lib.F32, stream())
    assert "exceed the fixed scratch" in str(e.value)
