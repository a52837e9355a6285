"""Parity of every op of the C ABI (called through mytorch_b200.fused_ops, i.e.
ctypes -> libmytorch_b200.so) against the NumPy oracle on the same seeded
inputs. Tolerances: fp32 1e-4, fp16/bf16 1e-2, relative to the largest
magnitude of the expected tensor (the path's stated per-op bars). Half cases
use the fp32 oracle evaluated on half-rounded inputs."""
import numpy as np
import pytest

from oracle import ops as O

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "float16", "bfloat16"]
TOL = {"float32": 1e-4, "float16": 1e-2, "bfloat16": 2e-2}


@pytest.fixture(scope="module")
def mt():
    import mytorch_b200 as m
    return m


def rnd(a, dtype):
    """Round host data to the device dtype, returned as fp32."""
    from mytorch_b200.array import f32_to_bf16_bits, bf16_bits_to_f32
    a = np.asarray(a, dtype=np.float32)
    if dtype == "float16":
        return a.astype(np.float16).astype(np.float32)
    if dtype == "bfloat16":
        return bf16_bits_to_f32(f32_to_bf16_bits(a)).reshape(a.shape)
    return a


def dev(mt, a, dtype):
    return mt.DeviceArray.from_numpy(a, dtype)


def close(got, want, rel, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    scale = max(np.abs(want).max(), 1e-3)   # an all-zero expectation is compared absolutely
    err = np.abs(got - want).max() / scale
    assert err <= rel, f"{what}: max err {err:.3e} (scale {scale:.3e}) > {rel}"


def no_device_flag(mt):
    import ctypes
    f = ctypes.c_int(0)
    mt._lib.device_flag_read(ctypes.byref(f), mt.stream())
    assert f.value == 0, f"device status word = {f.value}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(37, 96), (64, 768), (5, 1000), (130, 2048), (3, 52)])
@pytest.mark.parametrize("bias", [True, False])
def test_layernorm(mt, dtype, shape, bias):
    F = mt.fused_ops
    r = np.random.default_rng(1)
    x, g, b, dy = (rnd(r.standard_normal(s), dtype) for s in (shape, shape[1:], shape[1:], shape))
    y, mu, rs = O.layernorm_fwd(x, g, b if bias else None)
    dx, dg, db = O.layernorm_bwd(x, mu, rs, dy, g)
    dx_, dg_, db_ = None, None, None
    X, G, B, DY = dev(mt, x, dtype), dev(mt, g, dtype), dev(mt, b, dtype), dev(mt, dy, dtype)
    Y, MU, RS = F.fused_layernorm_forward(X, G, B if bias else None)
    DX, DG, DB = F.fused_layernorm_backward(X, MU, RS, DY, G, B if bias else None)
    t = TOL[dtype]
    close(Y.numpy(), y, t, "y"); close(MU.numpy(), mu, max(t, 1e-4) if dtype == "float32" else t, "mean")
    close(RS.numpy(), rs, t, "rstd"); close(DX.numpy(), dx, t, "dx")
    close(DG.numpy(), dg, 1e-4 if dtype == "float32" else t, "dgamma")
    if bias:
        close(DB.numpy(), db, 1e-4 if dtype == "float32" else t, "dbeta")
    # accumulate form adds into existing buffers; two runs are bit-identical
    acc = mt.DeviceArray.from_numpy(np.ones(shape[1], np.float32))
    F.fused_layernorm_backward(X, MU, RS, DY, G, None, dgamma_out=acc)
    close(acc.numpy(), dg + 1, 1e-4 if dtype == "float32" else t, "dgamma+=")
    DG2 = F.fused_layernorm_backward(X, MU, RS, DY, G, None)[1]
    assert np.array_equal(DG2.numpy(), DG.numpy())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(29, 128), (77, 1280), (9, 50)])
@pytest.mark.parametrize("weight", [True, False])
def test_rmsnorm(mt, dtype, shape, weight):
    F = mt.fused_ops
    r = np.random.default_rng(2)
    x, g, dy = (rnd(r.standard_normal(s), dtype) for s in (shape, shape[1:], shape))
    y, rs = O.rmsnorm_fwd(x, g if weight else None)
    dx, dg = O.rmsnorm_bwd(x, rs, dy, g if weight else None)
    X, G, DY = dev(mt, x, dtype), dev(mt, g, dtype), dev(mt, dy, dtype)
    Y, RS = F.fused_rmsnorm_forward(X, G if weight else None)
    DX, DG = F.fused_rmsnorm_backward(X, RS, DY, G if weight else None)
    t = TOL[dtype]
    close(Y.numpy(), y, t, "y"); close(RS.numpy(), rs, t, "rstd"); close(DX.numpy(), dx, t, "dx")
    if weight:
        close(DG.numpy(), dg, t, "dgamma")
    else:
        assert DG is None


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(33, 200), (64, 1024), (7, 4096), (5, 33)])
def test_softmax(mt, dtype, shape):
    F = mt.fused_ops
    r = np.random.default_rng(3)
    x, dy = rnd(r.standard_normal(shape), dtype), rnd(r.standard_normal(shape), dtype)
    s = O.softmax_fwd(x)
    S = F.fused_softmax_forward(dev(mt, x, dtype))
    close(S.numpy(), s, TOL[dtype], "softmax")
    s_r = rnd(s, dtype)
    DX = F.fused_softmax_backward(dev(mt, dy, dtype), dev(mt, s_r, dtype))
    close(DX.numpy(), O.softmax_bwd(dy, s_r), TOL[dtype], "softmax bwd")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["gelu", "relu_squared", "relu"])
def test_activations(mt, dtype, act):
    F = mt.fused_ops
    r = np.random.default_rng(4)
    x, dy = rnd(r.standard_normal((31, 1003)) * 2, dtype), rnd(r.standard_normal((31, 1003)), dtype)
    fwd = {"gelu": O.gelu_fwd, "relu_squared": O.relu2_fwd, "relu": lambda v: np.maximum(v, 0)}[act]
    bwd = {"gelu": O.gelu_bwd, "relu_squared": O.relu2_bwd, "relu": lambda v, d: (v > 0) * d}[act]
    close(F.fused_activation_forward(dev(mt, x, dtype), act).numpy(), fwd(x), TOL[dtype], act)
    close(F.fused_activation_backward(dev(mt, x, dtype), dev(mt, dy, dtype), act).numpy(), bwd(x, dy), TOL[dtype], act + " bwd")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,classes,ld", [(41, 131, 131), (64, 50257, 50264), (16, 50304, 50304), (3, 7, 16)])
def test_cross_entropy(mt, dtype, rows, classes, ld):
    F = mt.fused_ops
    r = np.random.default_rng(5)
    x = rnd(r.standard_normal((rows, classes)) * 2, dtype)
    y = r.integers(0, classes, rows).astype(np.int32)
    y[rows // 3] = -100
    buf = np.zeros((rows, ld), np.float32)
    buf[:, :classes] = x
    L = dev(mt, buf, dtype)
    Lv = mt.DeviceArray(L.ptr, (rows, classes), dtype, base=L)   # logical [rows, classes] view, row stride ld
    Y = mt.DeviceArray.from_numpy(y)
    loss, lse, tot = F.fused_cross_entropy_forward(Lv, Y, ld=ld, reduce=True)
    want_loss, want_lse = O.cross_entropy_rows(x, y)
    close(lse.numpy(), want_lse, 1e-5, "lse"); close(loss.numpy(), want_loss, 1e-4, "loss")
    t = tot.numpy()
    assert t[1] == rows - 1
    close(t[0] / t[1], O.cross_entropy_fwd(x, y), 1e-5, "mean loss")
    # backward over the logits, scale taken from device scalars (grad_output 3.0 / valid count)
    three = mt.DeviceArray.from_numpy(np.array([3.0], np.float32))
    cnt = mt.DeviceArray(tot.ptr + 4, (1,), "float32", base=tot)
    G = F.fused_cross_entropy_backward(Lv, Y, lse, scale=1.0, ld=ld, scale_dev=three, count_dev=cnt)
    assert G.ptr == L.ptr
    got = L.numpy()[:, :classes]
    close(got, O.cross_entropy_bwd(x, y, 3.0), 2e-2 if dtype != "float32" else 1e-4, "dlogits")
    assert np.all(got[rows // 3] == 0)
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(mt, dtype):
    F = mt.fused_ops
    r = np.random.default_rng(6)
    V, D = 97, 72
    w = rnd(r.standard_normal((V, D)), dtype)
    idx = r.integers(0, V, (6, 50)).astype(np.int32)
    idx[0, :20] = 5                      # a long run of one token
    dy = rnd(r.standard_normal((6, 50, D)), dtype)
    W, I, DY = dev(mt, w, dtype), mt.DeviceArray.from_numpy(idx), dev(mt, dy, dtype)
    close(F.fused_embedding_forward(W, I).numpy(), O.embedding_fwd(w, idx), 0.0, "gather")
    dw = F.fused_embedding_backward(DY, W, I)
    close(dw.numpy(), O.embedding_bwd(dy, idx, V), 1e-5, "scatter-add")
    dw2 = F.fused_embedding_backward(DY, W, I)
    assert np.array_equal(dw.numpy(), dw2.numpy()), "scatter-add must be reproducible"
    F.fused_embedding_backward(DY, W, I, out=dw)
    close(dw.numpy(), 2 * O.embedding_bwd(dy, idx, V), 1e-5, "scatter-add accumulate")
    no_device_flag(mt)


def test_embedding_empty_and_out_of_range(mt):
    import ctypes
    F = mt.fused_ops
    W = mt.DeviceArray.from_numpy(np.ones((4, 8), np.float32))
    out = F.fused_embedding_forward(W, mt.DeviceArray.from_numpy(np.zeros((0,), np.int32)))
    assert out.shape == (0, 8)
    out = F.fused_embedding_forward(W, mt.DeviceArray.from_numpy(np.array([1, 9], np.int32)))
    f = ctypes.c_int(0)
    mt._lib.device_flag_read(ctypes.byref(f), mt.stream())
    assert f.value == 1, "an out-of-range index must be recorded in the device status word"
    assert np.all(out.numpy()[1] == 0) and np.all(out.numpy()[0] == 1)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rope(mt, dtype):
    F = mt.fused_ops
    r = np.random.default_rng(7)
    B, T, H, D = 2, 19, 3, 32
    x, dy = rnd(r.standard_normal((B, T, H, D)), dtype), rnd(r.standard_normal((B, T, H, D)), dtype)
    cos, sin = O.rope_cos_sin(D, T)
    C_, S_ = mt.DeviceArray.from_numpy(cos), mt.DeviceArray.from_numpy(sin)
    X = dev(mt, x, dtype)
    F.fused_rope_forward(X, C_, S_)
    close(X.numpy(), O.rope_fwd(x, cos, sin), TOL[dtype], "rope")
    DY = dev(mt, dy, dtype)
    F.fused_rope_backward(DY, C_, S_)
    close(DY.numpy(), O.rope_bwd(dy, cos, sin), TOL[dtype], "rope bwd")


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (200, 136, 72), (1024, 768, 768), (64, 72, 40),
               (384, 2304, 768), (130, 520, 1032), (8, 8, 8), (1, 24, 16)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm(mt, dtype, ta, tb, M, N, K):
    F = mt.fused_ops
    r = np.random.default_rng(8)
    a = rnd(r.standard_normal((K, M) if ta else (M, K)), dtype)
    b = rnd(r.standard_normal((N, K) if tb else (K, N)), dtype)
    want = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64)
    C = F.gemm(dev(mt, a, dtype), dev(mt, b, dtype), trans_a=bool(ta), trans_b=bool(tb))
    close(C.numpy(), want, TOL[dtype], "gemm")
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_gemm_epilogues_and_fp32_out(mt, dtype):
    F = mt.fused_ops
    r = np.random.default_rng(9)
    M, N, K = 300, 264, 200
    x, w, b = rnd(r.standard_normal((M, K)), dtype), rnd(r.standard_normal((N, K)) * 0.1, dtype), rnd(r.standard_normal(N), dtype)
    pre = x @ w.T + b
    X, W, B = dev(mt, x, dtype), dev(mt, w, dtype), dev(mt, b, dtype)
    for act, f in (("gelu", O.gelu_fwd), ("relu_squared", O.relu2_fwd), (None, lambda v: v)):
        out, p = F.gemm(X, W, trans_b=True, bias=B, act=act, preact=True)
        close(p.numpy(), pre, TOL[dtype], "preact"); close(out.numpy(), f(pre), TOL[dtype], f"act {act}")
    # fp32 output, overwrite then read-modify-write then split-K atomic accumulation
    acc = F.gemm(X, W, trans_b=True, out_dtype="float32")
    close(acc.numpy(), x @ w.T, 1e-3, "fp32 out")
    F.gemm(X, W, trans_b=True, out=acc, accumulate=1)
    close(acc.numpy(), 2 * (x @ w.T), 1e-3, "accumulate=1")
    dy = rnd(r.standard_normal((4096, 136)), dtype)
    xx = rnd(r.standard_normal((4096, 200)), dtype)
    g = mt.DeviceArray.from_numpy(np.ones((136, 200), np.float32))
    F.gemm(dev(mt, dy, dtype), dev(mt, xx, dtype), trans_a=True, out=g, accumulate=2)
    close(g.numpy(), 1 + dy.T.astype(np.float64) @ xx, 1e-3, "split-K wgrad")
    # the reference-shaped entry points
    pre_, post_ = F.fused_linear_forward(X, dev(mt, np.ascontiguousarray(w.T), dtype), B, "gelu")
    close(pre_.numpy(), pre, TOL[dtype], "fused_linear pre"); close(post_.numpy(), O.gelu_fwd(pre), TOL[dtype], "fused_linear post")
    no_device_flag(mt)


def test_gemm_tensor_core_matches_cuda_core_kernel(mt):
    """Same fp16 inputs through both device kernels: differences are only
    accumulation order (fp32), far below the fp16 output rounding."""
    F = mt.fused_ops
    r = np.random.default_rng(10)
    a = mt.DeviceArray.from_numpy(r.standard_normal((512, 384)), "float16")
    b = mt.DeviceArray.from_numpy(r.standard_normal((640, 384)), "float16")
    tc = F.gemm(a, b, trans_b=True, out_dtype="float32").numpy()
    mt._lib.gemm_force_simt(1)
    try:
        cc = F.gemm(a, b, trans_b=True, out_dtype="float32").numpy()
    finally:
        mt._lib.gemm_force_simt(0)
    close(tc, cc, 1e-5, "tcgen05 vs CUDA-core")


@pytest.fixture
def cta_pairs(mt):
    """Forces the 256-row tiles shared by a pair of CTAs for the test's duration."""
    mt._lib.gemm_tile_policy(2)
    yield
    mt._lib.gemm_tile_policy(0)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(256, 512, 128), (200, 136, 72), (1024, 768, 768), (384, 2304, 768),
                                   (130, 520, 1032), (513, 300, 200), (2048, 3072, 768), (4096, 264, 64)])
def test_gemm_cta_pairs(mt, cta_pairs, dtype, ta, tb, M, N, K):
    """Same cases through the cta_group::2 kernel: ragged last row pair (the
    second CTA's rows partly or wholly past M), ragged N, every operand layout."""
    F = mt.fused_ops
    r = np.random.default_rng(13)
    a = rnd(r.standard_normal((K, M) if ta else (M, K)), dtype)
    b = rnd(r.standard_normal((N, K) if tb else (K, N)), dtype)
    want = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64)
    C = F.gemm(dev(mt, a, dtype), dev(mt, b, dtype), trans_a=bool(ta), trans_b=bool(tb))
    close(C.numpy(), want, TOL[dtype], "gemm, CTA pairs")
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_gemm_cta_pairs_epilogues_and_split_k(mt, cta_pairs, dtype):
    F = mt.fused_ops
    r = np.random.default_rng(14)
    M, N, K = 600, 264, 200
    x, w, b = rnd(r.standard_normal((M, K)), dtype), rnd(r.standard_normal((N, K)) * 0.1, dtype), rnd(r.standard_normal(N), dtype)
    pre = x @ w.T + b
    X, W, B = dev(mt, x, dtype), dev(mt, w, dtype), dev(mt, b, dtype)
    out, p = F.gemm(X, W, trans_b=True, bias=B, act="gelu", preact=True)
    close(p.numpy(), pre, TOL[dtype], "preact"); close(out.numpy(), O.gelu_fwd(pre), TOL[dtype], "gelu")
    dy = rnd(r.standard_normal((8192, 520)), dtype)
    xx = rnd(r.standard_normal((8192, 200)), dtype)
    g = mt.DeviceArray.from_numpy(np.ones((520, 200), np.float32))
    F.gemm(dev(mt, dy, dtype), dev(mt, xx, dtype), trans_a=True, out=g, accumulate=2)
    close(g.numpy(), 1 + dy.T.astype(np.float64) @ xx, 1e-3, "split-K wgrad, CTA pairs")
    # both tile shapes accumulate every output in the same order
    A2, B2 = dev(mt, rnd(r.standard_normal((1024, 512)), dtype), dtype), dev(mt, rnd(r.standard_normal((768, 512)), dtype), dtype)
    two = F.gemm(A2, B2, trans_b=True, out_dtype="float32").numpy()
    mt._lib.gemm_tile_policy(1)
    one = F.gemm(A2, B2, trans_b=True, out_dtype="float32").numpy()
    assert np.array_equal(one, two)
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,H,S,D,causal", [(2, 3, 70, 32, True), (1, 2, 128, 64, True), (2, 2, 257, 64, True),
                                            (1, 2, 100, 128, True), (1, 2, 64, 64, False), (1, 1, 1, 64, True),
                                            (1, 2, 33, 64, False), (2, 4, 1024, 64, True), (1, 2, 300, 128, False),
                                            (1, 3, 640, 128, True), (2, 2, 512, 64, False)])
def test_attention(mt, dtype, B, H, S, D, causal):
    F = mt.fused_ops
    r = np.random.default_rng(11)
    q, k, v, do = (rnd(r.standard_normal((B, H, S, D)), dtype) for _ in range(4))
    o, p = O.attention_fwd(q, k, v, causal=causal)
    dq, dk, dv = O.attention_bwd(q, k, v, p, do)
    Q, K, V, DO = (dev(mt, t, dtype) for t in (q, k, v, do))
    _, _, _, Ou, M = F.fused_sdpa_forward(Q, K, V, causal=causal)
    t = TOL[dtype]
    close(Ou.numpy(), o, t, "o")
    s = np.einsum("bhid,bhjd->bhij", q, k) / np.sqrt(D)
    if causal:
        s = s + np.triu(np.full((S, S), -np.inf), 1)
    lse = np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)
    close(M.numpy(), lse, 1e-3 if dtype != "float32" else 1e-5, "lse")
    DQ, DK, DV = F.fused_sdpa_backward(DO, Q, K, V, Ou, M, causal=causal)
    close(DQ.numpy(), dq, 2 * t, "dq"); close(DK.numpy(), dk, 2 * t, "dk"); close(DV.numpy(), dv, 2 * t, "dv")
    no_device_flag(mt)


@pytest.mark.parametrize("B,H,S,D", [(4, 18, 2048, 128), (6, 24, 2048, 64)])
def test_attention_head_grouped_tile_order_matches_cuda_core_kernels(mt, B, H, S, D):
    """Shapes large enough that the tensor-core kernels take the heads in groups (the forward
    once K and V of all heads exceed 64 MB: both shapes; the backward once its footprint
    exceeds 200 MB: the first) and that every persistent CTA takes many tiles from the global
    counter: every tile must still be visited exactly once. The CUDA-core kernels, which walk
    the tiles in plain order, are the reference; dQ/dK/dV would be off by whole tiles if one
    were skipped or done twice."""
    F = mt.fused_ops
    r = np.random.default_rng(21)
    Q, K, V, DO = (mt.DeviceArray.from_numpy(r.standard_normal((B, H, S, D)).astype(np.float32), "float16") for _ in range(4))
    _, _, _, o_tc, m_tc = F.fused_sdpa_forward(Q, K, V, causal=True)
    dq_tc, dk_tc, dv_tc = F.fused_sdpa_backward(DO, Q, K, V, o_tc, m_tc, causal=True)
    mt._lib.attn_force_simt(1)
    try:
        _, _, _, o_cc, m_cc = F.fused_sdpa_forward(Q, K, V, causal=True)
        dq_cc, dk_cc, dv_cc = F.fused_sdpa_backward(DO, Q, K, V, o_cc, m_cc, causal=True)
    finally:
        mt._lib.attn_force_simt(0)
    t = TOL["float16"]
    close(o_tc.numpy(), o_cc.numpy(), t, "o"); close(m_tc.numpy(), m_cc.numpy(), 1e-3, "lse")
    close(dq_tc.numpy(), dq_cc.numpy(), 2 * t, "dq"); close(dk_tc.numpy(), dk_cc.numpy(), 2 * t, "dk")
    close(dv_tc.numpy(), dv_cc.numpy(), 2 * t, "dv")
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("B,T,H,D", [(2, 257, 3, 64), (1, 1000, 2, 64), (2, 257, 2, 128), (1, 1000, 3, 128), (2, 1024, 12, 64)])
def test_attention_on_strided_projection_layouts(mt, dtype, B, T, H, D):
    """The tensor-core kernels reading q, k, v in place from the two layouts the models use — the
    per-head interleaved [q|k|v] projection of GPT-2 (F.qkv_attention) and separate [B,T,H,D]
    projections (F.bthd_attention) — at ragged and full sequence lengths, forward and backward."""
    Fn = mt.nn.functional
    r = np.random.default_rng(21)
    E = H * D
    qkv = rnd(r.standard_normal((B, T, H, 3 * D)), dtype)
    do = rnd(r.standard_normal((B, T, E)), dtype)
    q, k, v = (np.ascontiguousarray(qkv[..., i * D:(i + 1) * D].transpose(0, 2, 1, 3)) for i in range(3))   # [B,H,T,D]
    o, p = O.attention_fwd(q, k, v, causal=True)
    dq, dk, dv = O.attention_bwd(q, k, v, p, do.reshape(B, T, H, D).transpose(0, 2, 1, 3))
    want_o = o.transpose(0, 2, 1, 3).reshape(B, T, E)
    want_dqkv = np.concatenate([g.transpose(0, 2, 1, 3) for g in (dq, dk, dv)], axis=-1).reshape(B, T, 3 * E)
    t = TOL[dtype]
    # GPT-2 layout
    x = mt.Tensor(dev(mt, qkv.reshape(B, T, 3 * E), dtype), requires_grad=True)
    out = Fn.qkv_attention(x, H, is_causal=True)
    close(out.numpy(), want_o, t, "qkv_attention o")
    out.backward(dev(mt, do, dtype))
    close(x.grad.numpy(), want_dqkv, 2 * t, "qkv_attention dqkv")
    # separate projections, [B,T,H,D]
    bthd = [mt.Tensor(dev(mt, np.ascontiguousarray(a.transpose(0, 2, 1, 3)), dtype), requires_grad=True) for a in (q, k, v)]
    out2 = Fn.bthd_attention(*bthd, is_causal=True)
    close(out2.numpy(), want_o, t, "bthd_attention o")
    out2.backward(dev(mt, do, dtype))
    for a, g, name in zip(bthd, (dq, dk, dv), "qkv"):
        close(a.grad.numpy(), g.transpose(0, 2, 1, 3), 2 * t, f"bthd_attention d{name}")
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,T,H,D", [(2, 19, 3, 32), (1, 33, 10, 128), (2, 64, 5, 64), (1, 7, 1, 128)])
def test_rope_then_qk_rmsnorm_fused(mt, dtype, B, T, H, D):
    """rotary embedding followed by the parameter-free RMSNorm over head_dim on q and k, one kernel
    each way, against the oracle's separate ops chained the way the nanochat attention does; also
    through autograd (F.rope_qk_norm) with only one of the two outputs used."""
    F, Fn = mt.fused_ops, mt.nn.functional
    r = np.random.default_rng(31)
    q, k, dq_out, dk_out = (rnd(r.standard_normal((B, T, H, D)), dtype) for _ in range(4))
    cos, sin = O.rope_cos_sin(D, T)
    want, wgrad = [], []
    for x, dy in ((q, dq_out), (k, dk_out)):
        xr = O.rope_fwd(x, cos, sin).reshape(-1, D)
        y, rstd = O.rmsnorm_fwd(xr)
        dxr, _ = O.rmsnorm_bwd(xr, rstd, dy.reshape(-1, D))
        want.append((y.reshape(B, T, H, D), rstd))
        wgrad.append(O.rope_bwd(dxr.reshape(B, T, H, D), cos, sin))
    C_, S_ = dev(mt, cos, "float32"), dev(mt, sin, "float32")
    Q, Kk = dev(mt, q, dtype), dev(mt, k, dtype)
    yq, yk, rq, rk = F.fused_rope_rmsnorm_forward(Q, Kk, C_, S_)
    t = TOL[dtype]
    close(yq.numpy(), want[0][0], t, "q'"); close(yk.numpy(), want[1][0], t, "k'")
    close(rq.numpy(), want[0][1].reshape(-1), 1e-4 if dtype == "float32" else 5e-3, "rstd q")
    close(rk.numpy(), want[1][1].reshape(-1), 1e-4 if dtype == "float32" else 5e-3, "rstd k")
    gq, gk = F.fused_rope_rmsnorm_backward(dev(mt, dq_out, dtype), dev(mt, dk_out, dtype), yq, yk, rq, rk, C_, S_)
    close(gq.numpy(), wgrad[0], 2 * t, "dq"); close(gk.numpy(), wgrad[1], 2 * t, "dk")
    # autograd: both outputs used, then only the second
    qt, kt = mt.Tensor(Q, requires_grad=True), mt.Tensor(Kk, requires_grad=True)
    oq, ok = Fn.rope_qk_norm(qt, kt, C_, S_)
    tot = oq + ok
    tot.backward(dev(mt, dq_out, dtype))
    ref_q = O.rope_bwd(O.rmsnorm_bwd(O.rope_fwd(q, cos, sin).reshape(-1, D), want[0][1], dq_out.reshape(-1, D))[0].reshape(B, T, H, D), cos, sin)
    ref_k = O.rope_bwd(O.rmsnorm_bwd(O.rope_fwd(k, cos, sin).reshape(-1, D), want[1][1], dq_out.reshape(-1, D))[0].reshape(B, T, H, D), cos, sin)
    close(qt.grad.numpy(), ref_q, 2 * t, "autograd dq"); close(kt.grad.numpy(), ref_k, 2 * t, "autograd dk")
    qt2, kt2 = mt.Tensor(Q, requires_grad=True), mt.Tensor(Kk, requires_grad=True)
    _, ok2 = Fn.rope_qk_norm(qt2, kt2, C_, S_)
    ok2.backward(dev(mt, dk_out, dtype))
    close(kt2.grad.numpy(), wgrad[1], 2 * t, "autograd dk alone")
    assert not np.any(qt2.grad.numpy())
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,H,Hkv,S,D,causal", [(2, 4, 2, 70, 32, True), (1, 6, 2, 257, 64, True), (2, 4, 1, 128, 64, False),
                                                (1, 10, 5, 300, 128, True), (2, 8, 2, 1024, 64, True)])
def test_grouped_query_attention(mt, dtype, B, H, Hkv, S, D, causal):
    """Fewer key/value heads than query heads (fused_ops/flash_attention.py:445-455): query head h
    attends to key/value head h // (H // Hkv); dK and dV sum over the query heads of their group.
    Against the oracle with the key/value heads repeated, contiguous [B,H,S,D] and the models'
    [B,T,H,D] layout."""
    F, Fn = mt.fused_ops, mt.nn.functional
    r = np.random.default_rng(17)
    G = H // Hkv
    q, do = (rnd(r.standard_normal((B, H, S, D)), dtype) for _ in range(2))
    k, v = (rnd(r.standard_normal((B, Hkv, S, D)), dtype) for _ in range(2))
    o, p = O.attention_fwd(q, np.repeat(k, G, axis=1), np.repeat(v, G, axis=1), causal=causal)
    dq, dk, dv = O.attention_bwd(q, np.repeat(k, G, axis=1), np.repeat(v, G, axis=1), p, do)
    dk, dv = (g.reshape(B, Hkv, G, S, D).sum(axis=2) for g in (dk, dv))
    t = TOL[dtype]
    Q, K, V, DO = (dev(mt, a, dtype) for a in (q, k, v, do))
    _, _, _, Ou, M = F.fused_sdpa_forward(Q, K, V, causal=causal)
    close(Ou.numpy(), o, t, "o")
    DQ, DK, DV = F.fused_sdpa_backward(DO, Q, K, V, Ou, M, causal=causal)
    assert DK.shape == (B, Hkv, S, D) and DV.shape == (B, Hkv, S, D)
    close(DQ.numpy(), dq, 2 * t, "dq"); close(DK.numpy(), dk, 2 * t, "dk"); close(DV.numpy(), dv, 2 * t, "dv")
    if causal:   # the [B,T,H,D] form the nanochat model uses, through autograd
        ts = [mt.Tensor(dev(mt, np.ascontiguousarray(a.transpose(0, 2, 1, 3)), dtype), requires_grad=True) for a in (q, k, v)]
        out = Fn.bthd_attention(*ts, is_causal=True)
        close(out.numpy(), o.transpose(0, 2, 1, 3).reshape(B, S, H * D), t, "bthd o")
        out.backward(dev(mt, np.ascontiguousarray(do.transpose(0, 2, 1, 3)).reshape(B, S, H * D), dtype))
        for a, g, name in zip(ts, (dq, dk, dv), "qkv"):
            close(a.grad.numpy(), g.transpose(0, 2, 1, 3), 2 * t, f"bthd d{name}")
    no_device_flag(mt)


def test_attention_rejects_mismatched_key_value_shapes(mt):
    """Key/value heads that do not divide the query heads, fewer of them without enable_gqa, or
    another key length are refused on the host: the kernels index K and V with Q's extents."""
    Fn = mt.nn.functional
    q = mt.Tensor(mt.DeviceArray.zeros((1, 4, 64, 64), "float16"))
    kv = mt.Tensor(mt.DeviceArray.zeros((1, 2, 64, 64), "float16"))
    kv3 = mt.Tensor(mt.DeviceArray.zeros((1, 3, 64, 64), "float16"))
    with pytest.raises(ValueError):
        Fn.scaled_dot_product_attention(q, kv, kv, is_causal=True)          # needs enable_gqa=True
    assert Fn.scaled_dot_product_attention(q, kv, kv, is_causal=True, enable_gqa=True).shape == (1, 4, 64, 64)
    with pytest.raises(NotImplementedError):
        Fn.scaled_dot_product_attention(q, kv3, kv3, is_causal=True, enable_gqa=True)
    with pytest.raises(NotImplementedError):
        mt.fused_ops.fused_sdpa_forward(q.data, kv3.data, kv3.data, causal=True)
    longer = mt.Tensor(mt.DeviceArray.zeros((1, 128, 4, 64), "float16"))
    short = mt.Tensor(mt.DeviceArray.zeros((1, 64, 4, 64), "float16"))
    with pytest.raises(NotImplementedError):
        Fn.bthd_attention(short, longer, longer)


def test_embedding_backward_with_out_of_range_ids_between_equal_ids(mt):
    """Invalid ids (which the forward pass flags and the backward skips) must not split a run of
    equal valid ids between two warps: the sums of the valid rows stay exact."""
    F = mt.fused_ops
    r = np.random.default_rng(5)
    V, Dm, n = 300, 64, 4096
    idx = r.integers(0, 8, n).astype(np.int32)          # long runs of a few ids
    bad = r.choice(n, 200, replace=False)
    idx[bad[:100]] = -1
    idx[bad[100:150]] = V + 5
    idx[bad[150:]] = (1 << 16) + 3                      # low bits look like a valid id
    dy = r.standard_normal((n, Dm)).astype(np.float32)
    w = mt.DeviceArray.zeros((V, Dm), "float32")
    got = F.fused_embedding_backward(dev(mt, dy, "float32"), w, dev(mt, idx, "int32")).numpy()
    ok = (idx >= 0) & (idx < V)
    want = np.zeros((V, Dm), np.float64)
    np.add.at(want, idx[ok], dy[ok].astype(np.float64))
    close(got, want, 1e-5, "dW with invalid ids")


def test_golden_small_vectors_fp32(mt, golden_ops, op_inputs):
    """The committed reference outputs, fp32, through the library."""
    F = mt.fused_ops
    d, g = op_inputs, golden_ops
    D = lambda a: mt.DeviceArray.from_numpy(a)
    X, G, B = D(d["ln_x"]), D(d["ln_g"]), D(d["ln_b"])
    Y, MU, RS = F.fused_layernorm_forward(X, G, B)
    DX, DG, DB = F.fused_layernorm_backward(X, MU, RS, D(d["ln_dy"]), G, B)
    close(Y.numpy(), g["ln_y"], 1e-4); close(DX.numpy(), g["ln_dx"], 1e-4)
    close(DG.numpy(), g["ln_dg"], 1e-4); close(DB.numpy(), g["ln_db"], 1e-4)
    Y, RS = F.fused_rmsnorm_forward(D(d["rms_x"]), D(d["rms_g"]))
    close(Y.numpy(), g["rms_y"], 1e-4)
    close(F.fused_softmax_forward(D(d["sm_x"])).numpy(), g["sm_y"], 1e-4)
    close(F.gemm(D(d["lin_x"]), D(d["lin_w"]), trans_b=True, bias=D(d["lin_b"])).numpy(), g["lin_y"], 1e-4)
    close(F.gemm(D(d["lin_dy"]), D(d["lin_w"])).numpy(), g["lin_dx"], 1e-4)
    close(F.gemm(D(d["lin_dy"]), D(d["lin_x"]), trans_a=True).numpy(), g["lin_dw"], 1e-4)
    close(F.fused_activation_forward(D(d["act_x"]), "gelu").numpy(), g["gelu_y"], 1e-4)
    close(F.fused_activation_backward(D(d["act_x"]), D(d["act_dy"]), "gelu").numpy(), g["gelu_dx"], 1e-4)
    close(F.fused_activation_backward(D(d["act_x"]), D(d["act_dy"]), "relu_squared").numpy(), g["relu2_dx"], 1e-4)
    L = D(d["ce_x"]); Yl = D(d["ce_y"])
    loss, lse, tot = F.fused_cross_entropy_forward(L, Yl, reduce=True)
    t = tot.numpy()
    close(t[0] / t[1], g["ce_loss"], 1e-5)
    F.fused_cross_entropy_backward(L, Yl, lse, scale=1.0 / t[1])
    close(L.numpy(), g["ce_dx"], 1e-4)
    close(F.fused_embedding_backward(D(d["emb_dy"]), D(d["emb_w"]), D(d["emb_idx"])).numpy(), g["emb_dw"], 1e-5)
    Q, K, V = D(d["at_q"]), D(d["at_k"]), D(d["at_v"])
    _, _, _, Ou, M = F.fused_sdpa_forward(Q, K, V, causal=True)
    close(Ou.numpy(), g["at_o"], 1e-4)
    DQ, DK, DV = F.fused_sdpa_backward(D(d["at_do"]), Q, K, V, Ou, M, causal=True)
    close(DQ.numpy(), g["at_dq"], 1e-4); close(DK.numpy(), g["at_dk"], 1e-4); close(DV.numpy(), g["at_dv"], 1e-4)
    Xr = D(d["rope_x"])
    F.fused_rope_forward(Xr, D(g["rope_cos"]), D(g["rope_sin"]))
    close(Xr.numpy(), g["rope_y"], 1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gemm_aux_operand_residual_and_activation_backward(mt, dtype):
    """mt_gemm_ex: result combined with an [M,N] operand in the epilogue."""
    F = mt.fused_ops
    r = np.random.default_rng(12)
    M, N, K = 200, 264, 136
    a, b, aux = rnd(r.standard_normal((M, K)), dtype), rnd(r.standard_normal((N, K)) * 0.2, dtype), rnd(r.standard_normal((M, N)), dtype)
    base = a.astype(np.float64) @ b.T.astype(np.float64)
    A, B, AUX = dev(mt, a, dtype), dev(mt, b, dtype), dev(mt, aux, dtype)
    t = TOL[dtype]
    close(F.gemm(A, B, trans_b=True, aux=AUX, aux_mode=1).numpy(), base + aux, t, "residual")
    close(F.gemm(A, B, trans_b=True, aux=AUX, aux_mode=2).numpy(), O.gelu_bwd(aux.astype(np.float64), base), 2 * t, "gelu'")
    close(F.gemm(A, B, trans_b=True, aux=AUX, aux_mode=3).numpy(), O.relu2_bwd(aux.astype(np.float64), base), 2 * t, "relu2'")
    close(F.gemm(A, B, trans_b=True, aux=AUX, aux_mode=4).numpy(), (aux > 0) * base, 2 * t, "relu'")
    # relu_squared's derivative recovered from its OUTPUT: aux = relu(u)^2, factor 2*sqrt(aux) = 2*relu(u)
    h = rnd(np.maximum(aux, 0.0) ** 2, dtype)
    close(F.gemm(A, B, trans_b=True, aux=dev(mt, h, dtype), aux_mode=6).numpy(), base * 2.0 * np.sqrt(h.astype(np.float64)),
          2 * t, "relu2' from its output")
    # activation first, then the residual
    close(F.gemm(A, B, trans_b=True, act="gelu", aux=AUX, aux_mode=1).numpy(), O.gelu_fwd(base) + aux, t, "gelu + residual")
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(64, 768), (5, 1000), (3, 52)])
def test_norm_backward_adds_into_existing_dx(mt, dtype, shape):
    F = mt.fused_ops
    r = np.random.default_rng(13)
    x, g, dy, prev = (rnd(r.standard_normal(s), dtype) for s in (shape, shape[1:], shape, shape))
    _, mu, rs = O.layernorm_fwd(x, g, None)
    want = O.layernorm_bwd(x, mu, rs, dy, g)[0] + prev
    X, G, DY, PREV = dev(mt, x, dtype), dev(mt, g, dtype), dev(mt, dy, dtype), dev(mt, prev, dtype)
    _, MU, RS = F.fused_layernorm_forward(X, G, None)
    DX, _, _ = F.fused_layernorm_backward(X, MU, RS, DY, G, None, dx_out=PREV)
    assert DX.ptr == PREV.ptr
    close(PREV.numpy(), want, 2 * TOL[dtype], "layernorm dx +=")
    _, rs2 = O.rmsnorm_fwd(x, None)
    want = O.rmsnorm_bwd(x, rs2, dy, None)[0] + prev
    PREV2 = dev(mt, prev, dtype)
    _, RS2 = F.fused_rmsnorm_forward(X, None)
    F.fused_rmsnorm_backward(X, RS2, DY, None, dx_out=PREV2)
    close(PREV2.numpy(), want, 2 * TOL[dtype], "rmsnorm dx +=")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [64, 128])
def test_kv_cache_append_and_decode_attention(mt, dtype, D):
    """mt_kv_append into a ring cache (including the wrap that overwrites the oldest rows) and
    mt_attn_decode of a few query rows over it, against NumPy softmax attention."""
    _lib = mt._lib
    from mytorch_b200.array import stream
    r = np.random.default_rng(15)
    B, H, MAXL = 2, 3, 48
    S3 = _lib.Strides3
    kc = mt.DeviceArray.zeros((B, H, MAXL, D), dtype)
    vc = mt.DeviceArray.zeros((B, H, MAXL, D), dtype)
    sc = S3(H * MAXL * D, MAXL * D, D)
    ring_k = np.zeros((B, H, MAXL, D)); ring_v = np.zeros((B, H, MAXL, D))
    appended = 0
    for n_new in (20, 1, 17, 1, 30):                 # 69 rows into a ring of 48
        k = rnd(r.standard_normal((B, H, n_new, D)), dtype); v = rnd(r.standard_normal((B, H, n_new, D)), dtype)
        K_, V_ = dev(mt, k, dtype), dev(mt, v, dtype)
        sn = S3(H * n_new * D, n_new * D, D)
        _lib.kv_append(K_.ptr, V_.ptr, kc.ptr, vc.ptr, sn, sn, sc, B, H, n_new, appended % MAXL, MAXL, D, kc.code, stream())
        for i in range(n_new):
            ring_k[:, :, (appended + i) % MAXL] = k[:, :, i]; ring_v[:, :, (appended + i) % MAXL] = v[:, :, i]
        appended += n_new
        kv_len = min(appended, MAXL)
        close(kc.numpy(), ring_k, 1e-6, "ring k"); close(vc.numpy(), ring_v, 1e-6, "ring v")
        for q_len, causal_offset in ((1, -1), (3, -1), (2, kv_len - 2)):
            q = rnd(r.standard_normal((B, H, q_len, D)), dtype)
            Q = dev(mt, q, dtype)
            out = mt.DeviceArray.empty((B, H, q_len, D), dtype)
            sq = S3(H * q_len * D, q_len * D, D)
            _lib.attn_decode(Q.ptr, kc.ptr, vc.ptr, out.ptr, sq, sc, sq, B, H, q_len, kv_len, D, D ** -0.5,
                             causal_offset, Q.code, stream())
            s = np.einsum("bhqd,bhkd->bhqk", q, ring_k[:, :, :kv_len]) / np.sqrt(D)
            if causal_offset >= 0:
                for i in range(q_len):
                    s[:, :, i, causal_offset + i + 1:] = -np.inf
            p = np.exp(s - s.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
            close(out.numpy(), np.einsum("bhqk,bhkd->bhqd", p, ring_v[:, :, :kv_len]), TOL[dtype], "decode attention")
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act,grad", [("gelu", lambda v: O.gelu_bwd(v, np.ones_like(v))),
                                      ("relu_squared", lambda v: O.relu2_bwd(v, np.ones_like(v)))])
@pytest.mark.parametrize("M,N,K", [(300, 264, 200), (513, 136, 72), (45, 50, 24)])
def test_gemm_stores_activation_derivative_and_multiplies_by_it(mt, dtype, act, grad, M, N, K):
    """MT_ACT_STORE_GRAD: the second output of the forward GEMM holds act'(x W^T + b); aux_mode 5
    multiplies a later GEMM's result by it - together the backward of the activation."""
    F = mt.fused_ops
    r = np.random.default_rng(16)
    x, w, b = rnd(r.standard_normal((M, K)), dtype), rnd(r.standard_normal((N, K)) * 0.2, dtype), rnd(r.standard_normal(N), dtype)
    pre = x.astype(np.float64) @ w.T + b
    X, W, B = dev(mt, x, dtype), dev(mt, w, dtype), dev(mt, b, dtype)
    fwd = {"gelu": O.gelu_fwd, "relu_squared": O.relu2_fwd}[act]
    t = TOL[dtype]
    for policy in (1, 2):
        mt._lib.gemm_tile_policy(policy)
        try:
            out, d = F.gemm(X, W, trans_b=True, bias=B, act=act, preact="grad")
        finally:
            mt._lib.gemm_tile_policy(0)
        close(out.numpy(), fwd(pre), t, f"{act} (policy {policy})")
        close(d.numpy(), grad(pre), 2 * t, f"{act}' (policy {policy})")
    dy, w2 = rnd(r.standard_normal((M, 40)), dtype), rnd(r.standard_normal((40, N)) * 0.3, dtype)
    dsaved = rnd(d.numpy(), dtype)
    got = F.gemm(dev(mt, dy, dtype), dev(mt, w2, dtype), aux=dev(mt, dsaved, dtype), aux_mode=5)
    close(got.numpy(), (dy.astype(np.float64) @ w2) * dsaved, t, "result * saved derivative")
    no_device_flag(mt)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,classes,ld,softcap", [(41, 131, 131, None), (64, 50257, 50264, None), (16, 50304, 50304, None),
                                                     (3, 7, 16, None), (20, 1000, 1000, 15.0),
                                                     (8, 4096, 4104, None), (5, 16, 16, None), (4, 24, 32, 15.0)])
def test_cross_entropy_forward_and_gradient_in_one_pass(mt, dtype, rows, classes, ld, softcap):
    """mt_ce_fwd_grad: same loss / lse / count as the forward kernel, and the logits buffer then
    holds the gradient of the mean loss times the announced upstream value."""
    F = mt.fused_ops
    r = np.random.default_rng(17)
    x = rnd(r.standard_normal((rows, classes)) * 2, dtype)
    y = r.integers(0, classes, rows).astype(np.int32)
    y[rows // 3] = -100
    buf = np.zeros((rows, ld), np.float32)
    buf[:, :classes] = x
    L = dev(mt, buf, dtype)
    Lv = mt.DeviceArray(L.ptr, (rows, classes), dtype, base=L)
    Y = mt.DeviceArray.from_numpy(y)
    up = mt.DeviceArray.from_numpy(np.array([3.0], np.float32))
    loss, lse, tot = F.fused_cross_entropy_forward_backward(Lv, Y, softcap, ld=ld, scale_dev=up)
    xs = x if softcap is None else softcap * np.tanh(x / softcap)
    want_loss, want_lse = O.cross_entropy_rows(xs, y)
    close(lse.numpy(), want_lse, 1e-5, "lse"); close(loss.numpy(), want_loss, 1e-4, "loss")
    t = tot.numpy()
    assert t[1] == rows - 1
    close(t[2], want_loss.sum() / (rows - 1), 1e-5, "mean loss")
    want = O.cross_entropy_bwd(xs, y, 3.0)
    if softcap is not None:
        want = want * (1.0 - np.tanh(x / softcap) ** 2)
    got = L.numpy()[:, :classes]
    close(got, want, 2e-2 if dtype != "float32" else 1e-4, "dlogits")
    assert np.all(got[rows // 3] == 0)
    no_device_flag(mt)


def test_empty_inputs_are_accepted_everywhere(mt):
    """Zero rows / zero batch: every entry point returns without launching on nothing and without
    touching the device status word (the reference's wrappers get such shapes from a last, short
    batch that a sharded loader can leave empty)."""
    F = mt.fused_ops
    Z = lambda *s, dt="float16": mt.DeviceArray.empty(s, dt)
    g = mt.DeviceArray.from_numpy(np.ones(64, np.float32), "float16")
    y, mu, rs = F.fused_layernorm_forward(Z(0, 64), g, None)
    assert y.shape == (0, 64) and mu.shape == (0,)
    dx, dg, _ = F.fused_layernorm_backward(Z(0, 64), mu, rs, Z(0, 64), g, None)
    assert dx.shape == (0, 64) and np.all(dg.numpy() == 0)
    y, rs = F.fused_rmsnorm_forward(Z(0, 64), None)
    assert y.shape == (0, 64)
    assert F.fused_softmax_forward(Z(0, 128)).shape == (0, 128)
    assert F.fused_activation_forward(Z(0, 32), "gelu").shape == (0, 32)
    assert F.gemm(Z(0, 64), Z(32, 64), trans_b=True).shape == (0, 32)
    assert F.gemm(Z(16, 64), Z(0, 64), trans_b=True).shape == (16, 0)
    w = mt.DeviceArray.from_numpy(np.ones((10, 8), np.float32), "float16")
    idx = mt.DeviceArray.empty((0, 5), "int32")
    assert F.fused_embedding_forward(w, idx).shape == (0, 5, 8)
    assert np.all(F.fused_embedding_backward(Z(0, 5, 8), w, idx).numpy() == 0)
    loss, lse = F.fused_cross_entropy_forward(Z(0, 100), mt.DeviceArray.empty((0,), "int32"))
    assert loss.shape == (0,)
    q = Z(0, 2, 128, 64)
    _, _, _, o, m = F.fused_sdpa_forward(q, q, q, causal=True)
    assert o.shape == (0, 2, 128, 64)
    dq, dk, dv = F.fused_sdpa_backward(q, q, q, q, o, m, causal=True)
    assert dq.shape == dk.shape == dv.shape == (0, 2, 128, 64)
    no_device_flag(mt)
