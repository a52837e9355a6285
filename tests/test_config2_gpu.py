"""The isolated fused-op suite at its stated shapes: every op forward and backward, in fp16 and
fp32, inputs drawn N(0,1) from seed 1, through the C ABI against the NumPy oracle.

  (a) causal attention  B=8, H=12, S=1024, D=64
  (b) LayerNorm         16384 x 768, gamma = 1, beta = 0
  (c) row softmax       16384 x 1024
  (d) cross entropy     8192 x 50304 logits, targets uniform in [0, 50257)
  (e) matmul            8192 x 768 x 3072 (as Linear: X[8192,768], W[3072,768])

The shape lists these come from are the reference's own numerical checks
(mytorch/nn/functional/fused_ops/benchmark.py:23-49 matmul, :111-138 softmax, :470-515
layernorm, :644-689 attention). Tolerances: fp32 1e-4, fp16 1e-2 of the largest expected
magnitude; the fp16 expectation is the fp32 oracle evaluated on fp16-rounded inputs."""
import numpy as np
import pytest

from oracle import ops as O

pytestmark = pytest.mark.gpu

DTYPES = ["float16", "float32"]
TOL = {"float32": 1e-4, "float16": 1e-2}


@pytest.fixture(scope="module")
def mt():
    import mytorch_b200 as m
    return m


def rnd(a, dtype):
    a = np.asarray(a, dtype=np.float32)
    return a.astype(np.float16).astype(np.float32) if dtype == "float16" else a


def close(got, want, rel, what):
    got = np.asarray(got, dtype=np.float32)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    scale = max(float(np.abs(want).max()), 1e-3)
    err = float(np.abs(got - want).max()) / scale
    assert err <= rel, f"{what}: max err {err:.3e} (scale {scale:.3e}) > {rel}"


def no_device_flag(mt):
    import ctypes
    f = ctypes.c_int(0)
    mt._lib.device_flag_read(ctypes.byref(f), mt.stream())
    assert f.value == 0, f"device status word = {f.value}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_8x12x1024x64_causal(mt, dtype):
    F = mt.fused_ops
    r = np.random.default_rng(1)
    B, H, S, D = 8, 12, 1024, 64
    q, k, v, do = (rnd(r.standard_normal((B, H, S, D), dtype=np.float32), dtype) for _ in range(4))
    o, p = O.attention_fwd(q, k, v, causal=True)
    dq, dk, dv = O.attention_bwd(q, k, v, p, do)
    Q, K, V, DO = (mt.DeviceArray.from_numpy(t, dtype) for t in (q, k, v, do))
    _, _, _, Ou, M = F.fused_sdpa_forward(Q, K, V, causal=True)
    t = TOL[dtype]
    close(Ou.numpy(), o, t, "o")
    DQ, DK, DV = F.fused_sdpa_backward(DO, Q, K, V, Ou, M, causal=True)
    close(DQ.numpy(), dq, 2 * t, "dq"); close(DK.numpy(), dk, 2 * t, "dk"); close(DV.numpy(), dv, 2 * t, "dv")
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", DTYPES)
def test_layernorm_16384x768(mt, dtype):
    F = mt.fused_ops
    r = np.random.default_rng(1)
    x = rnd(r.standard_normal((16384, 768), dtype=np.float32), dtype)
    dy = rnd(r.standard_normal((16384, 768), dtype=np.float32), dtype)
    g, b = np.ones(768, np.float32), np.zeros(768, np.float32)
    y, mean, rstd = O.layernorm_fwd(x, g, b)
    dx, dg, db = O.layernorm_bwd(x, mean, rstd, dy, g)
    X, G, Bt, DY = (mt.DeviceArray.from_numpy(a, dtype) for a in (x, g, b, dy))
    Y, MU, RS = F.fused_layernorm_forward(X, G, Bt)
    t = TOL[dtype]
    close(Y.numpy(), y, t, "y")
    close(MU.numpy(), mean.reshape(-1), 1e-4, "mean"); close(RS.numpy(), rstd.reshape(-1), 1e-4, "rstd")
    DX, DG, DB = F.fused_layernorm_backward(X, MU, RS, DY, G, Bt)
    close(DX.numpy(), dx, t, "dx")
    # column sums over 16384 rows: compared against the float64 sum of the same products
    close(DG.numpy(), dg.reshape(-1), 1e-4 if dtype == "float32" else 1e-3, "dgamma")
    close(DB.numpy(), db.reshape(-1), 1e-4 if dtype == "float32" else 1e-3, "dbeta")
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", DTYPES)
def test_softmax_16384x1024(mt, dtype):
    F = mt.fused_ops
    r = np.random.default_rng(1)
    x = rnd(r.standard_normal((16384, 1024), dtype=np.float32), dtype)
    dy = rnd(r.standard_normal((16384, 1024), dtype=np.float32), dtype)
    s = O.softmax_fwd(x)
    X, DY = mt.DeviceArray.from_numpy(x, dtype), mt.DeviceArray.from_numpy(dy, dtype)
    S = F.fused_softmax_forward(X)
    t = TOL[dtype]
    close(S.numpy(), s, t, "softmax")
    s_dev = S.numpy().astype(np.float32)            # the backward consumes the device's own (rounded) output
    close(F.fused_softmax_backward(DY, S).numpy(), O.softmax_bwd(dy, s_dev), t, "dx")
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", DTYPES)
def test_cross_entropy_8192x50304(mt, dtype):
    F = mt.fused_ops
    r = np.random.default_rng(1)
    N, C = 8192, 50304
    x = rnd(r.standard_normal((N, C), dtype=np.float32), dtype)
    y = r.integers(0, 50257, N).astype(np.int32)
    loss, lse = O.cross_entropy_rows(x, y)
    X, Y = mt.DeviceArray.from_numpy(x, dtype), mt.DeviceArray.from_numpy(y, "int32")
    L, LSE, tot = F.fused_cross_entropy_forward(X, Y, reduce=True)
    close(L.numpy(), loss, 1e-4 if dtype == "float32" else 1e-3, "loss rows")
    close(LSE.numpy(), lse, 1e-5 if dtype == "float32" else 1e-4, "lse")
    want_mean = float(loss.astype(np.float64).mean())
    assert abs(float(tot.numpy()[2]) - want_mean) <= 1e-5 * want_mean
    grad = O.cross_entropy_bwd(x, y, grad_output=1.0)
    # the mean's gradient carries 1/N: compared times N (scale 1, no count), which keeps fp16 in its normal range
    G = F.fused_cross_entropy_backward(X, Y, LSE, scale=1.0)
    got = G.numpy().astype(np.float32)
    close(got, grad * N, TOL[dtype], "dlogits (x N)")
    # forward+gradient in one pass gives the same two results
    X2 = mt.DeviceArray.from_numpy(x, dtype)
    L2, LSE2, tot2 = F.fused_cross_entropy_forward_backward(X2, Y, scale=float(N))
    close(L2.numpy(), loss, 1e-4 if dtype == "float32" else 1e-3, "loss rows (one pass)")
    close(X2.numpy().astype(np.float32), grad * N, TOL[dtype], "dlogits (one pass, x N)")
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", DTYPES)
def test_matmul_8192x768x3072(mt, dtype):
    F = mt.fused_ops
    r = np.random.default_rng(1)
    x = rnd(r.standard_normal((8192, 768), dtype=np.float32), dtype)
    w = rnd(r.standard_normal((3072, 768), dtype=np.float32), dtype)
    dy = rnd(r.standard_normal((8192, 3072), dtype=np.float32), dtype)
    X, W, DY = (mt.DeviceArray.from_numpy(a, dtype) for a in (x, w, dy))
    t = TOL[dtype]
    close(F.gemm(X, W, trans_b=True).numpy(), O.linear_fwd(x, w), t, "y = x w^T")
    dx, dw, _ = O.linear_bwd(x, w, dy)
    close(F.gemm(DY, W).numpy(), dx, t, "dx = dy w")
    close(F.gemm(DY, X, trans_a=True, out_dtype="float32").numpy(), dw, t if dtype == "float16" else 1e-4, "dw = dy^T x")
    close(F.fused_grouped_matmul(X, mt.DeviceArray.from_numpy(np.ascontiguousarray(w.T), dtype)).numpy(),
          O.linear_fwd(x, w), t, "fused_grouped_matmul")
    no_device_flag(mt)
