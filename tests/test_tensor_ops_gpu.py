"""The general-purpose Tensor ops (transpose, permute, chunk, slicing, elementwise arithmetic with
broadcasting, sums and means, matmul, concatenate, stack), forward and backward against NumPy,
and the reference's non-fused attention branch (gpt2_trainer/gpt2.py:168-203: reshape ->
transpose -> chunk -> q @ k^T / sqrt(D) + mask -> softmax -> @ v) written with them, against the
fused attention of the library and the oracle."""
import numpy as np
import pytest

from oracle import ops as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mt():
    import mytorch_b200 as m
    return m


def T(mt, a, grad=True):
    return mt.Tensor(np.asarray(a, dtype=np.float32), requires_grad=grad)


def close(got, want, tol=1e-5, what=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    scale = max(np.abs(want).max(), 1e-3) if want.size else 1.0
    assert np.abs(got - want).max() <= tol * scale if want.size else True, what


def test_transpose_and_permute(mt):
    r = np.random.default_rng(0)
    x = r.standard_normal((2, 3, 5, 4)).astype(np.float32)
    g = r.standard_normal((2, 5, 3, 4)).astype(np.float32)
    xt = T(mt, x)
    y = xt.transpose(1, 2)
    close(y.numpy(), x.transpose(0, 2, 1, 3))
    y.backward(mt.DeviceArray.from_numpy(g))
    close(xt.grad.numpy(), g.transpose(0, 2, 1, 3))
    xt = T(mt, x)
    y = mt.permute(xt, 3, 0, 2, 1)
    close(y.numpy(), x.transpose(3, 0, 2, 1))
    g2 = r.standard_normal(y.shape).astype(np.float32)
    y.backward(mt.DeviceArray.from_numpy(g2))
    close(xt.grad.numpy(), g2.transpose(1, 3, 2, 0))
    close(T(mt, x).transpose(-1, -2).numpy(), x.swapaxes(-1, -2))


def test_chunk_and_partial_use(mt):
    r = np.random.default_rng(1)
    x = r.standard_normal((2, 3, 5, 12)).astype(np.float32)
    xt = T(mt, x)
    a, b, c = mt.chunk(xt, 3, dim=-1)
    for got, want in zip((a, b, c), np.split(x, 3, axis=-1)):
        close(got.numpy(), want)
    g = r.standard_normal((2, 3, 5, 4)).astype(np.float32)
    (a + b * 2.0 + c * 3.0).backward(mt.DeviceArray.from_numpy(g))
    close(xt.grad.numpy(), np.concatenate([g, 2 * g, 3 * g], axis=-1))
    xt = T(mt, x)
    p = xt.chunk(5, dim=2)
    assert len(p) == 5 and p[3].shape == (2, 3, 1, 12)
    g = r.standard_normal(p[3].shape).astype(np.float32)
    p[3].backward(mt.DeviceArray.from_numpy(g))         # the other pieces receive nothing: their slices are zero
    want = np.zeros_like(x)
    want[:, :, 3:4] = g
    close(xt.grad.numpy(), want)
    with pytest.raises(ValueError):
        xt.chunk(5, dim=-1)


def test_getitem_slices(mt):
    r = np.random.default_rng(2)
    x = r.standard_normal((3, 4, 6, 8)).astype(np.float32)
    for idx in [np.s_[:, :, :5, :5], np.s_[1], np.s_[:, 1:3, ::2, 4], np.s_[..., -1], np.s_[2, :, 1:-1], np.s_[0:1, 0:1, :4, :4]]:
        xt = T(mt, x)
        y = xt[idx]
        close(y.numpy(), x[idx], what=str(idx))
        g = r.standard_normal(x[idx].shape).astype(np.float32)
        y.backward(mt.DeviceArray.from_numpy(g))
        want = np.zeros_like(x)
        want[idx] = g
        close(xt.grad.numpy(), want, what=str(idx))


def test_elementwise_with_broadcasting(mt):
    r = np.random.default_rng(3)
    a = r.standard_normal((2, 3, 4, 5)).astype(np.float32)
    b = r.standard_normal((1, 1, 4, 5)).astype(np.float32)
    g = r.standard_normal(a.shape).astype(np.float32)
    for op, f, ga, gb in [("add", lambda x, y: x + y, lambda: g, lambda: g.sum((0, 1), keepdims=True)),
                          ("sub", lambda x, y: x - y, lambda: g, lambda: -g.sum((0, 1), keepdims=True)),
                          ("mul", lambda x, y: x * y, lambda: g * b, lambda: (g * a).sum((0, 1), keepdims=True))]:
        at, bt = T(mt, a), T(mt, b)
        y = f(at, bt)
        close(y.numpy(), f(a, b), what=op)
        y.backward(mt.DeviceArray.from_numpy(g))
        close(at.grad.numpy(), ga(), what=op + " da")
        close(bt.grad.numpy(), gb(), 1e-5, op + " db")
    at = T(mt, a)
    y = -at
    y.backward(mt.DeviceArray.from_numpy(g))
    close(y.numpy(), -a); close(at.grad.numpy(), -g)
    same = T(mt, a) * T(mt, a, grad=False)
    close(same.numpy(), a * a)


@pytest.mark.parametrize("dim,keep", [(None, False), (None, True), (-1, False), (-1, True), (0, False), (1, True), (2, False)])
def test_sum_and_mean(mt, dim, keep):
    r = np.random.default_rng(4)
    x = r.standard_normal((3, 4, 5, 6)).astype(np.float32)
    for name in ("sum", "mean"):
        xt = T(mt, x)
        y = getattr(xt, name)(dim, keep)
        want = getattr(x.astype(np.float64), name)(axis=dim, keepdims=keep)
        close(y.numpy(), want, 1e-5, f"{name} {dim} {keep}")
        g = r.standard_normal(np.shape(want)).astype(np.float32)
        y.backward(mt.DeviceArray.from_numpy(g))
        gk = g.reshape(np.shape(getattr(x, name)(axis=dim, keepdims=True)))
        n = x.size if dim is None else x.shape[dim]
        close(xt.grad.numpy(), np.broadcast_to(gk, x.shape) / (n if name == "mean" else 1), 1e-5, f"{name} grad")


def test_matmul_batched_and_shared(mt):
    r = np.random.default_rng(5)
    a = r.standard_normal((2, 3, 7, 5)).astype(np.float32)
    b = r.standard_normal((2, 3, 5, 6)).astype(np.float32)
    g = r.standard_normal((2, 3, 7, 6)).astype(np.float32)
    at, bt = T(mt, a), T(mt, b)
    y = at @ bt
    close(y.numpy(), a @ b, 1e-5)
    y.backward(mt.DeviceArray.from_numpy(g))
    close(at.grad.numpy(), g @ b.swapaxes(-1, -2), 1e-5, "dA")
    close(bt.grad.numpy(), a.swapaxes(-1, -2) @ g, 1e-5, "dB")
    w = r.standard_normal((5, 9)).astype(np.float32)
    at, wt = T(mt, a), T(mt, w)
    y = at @ wt
    close(y.numpy(), a @ w, 1e-5)
    g2 = r.standard_normal(y.shape).astype(np.float32)
    y.backward(mt.DeviceArray.from_numpy(g2))
    close(at.grad.numpy(), g2 @ w.T, 1e-5, "dA shared")
    close(wt.grad.numpy(), np.einsum("bhmk,bhmn->kn", a, g2), 1e-5, "dW shared")
    with pytest.raises(ValueError):
        T(mt, a) @ T(mt, w.T)


def test_concatenate_and_stack(mt):
    r = np.random.default_rng(6)
    parts = [r.standard_normal((2, n, 4)).astype(np.float32) for n in (3, 1, 5)]
    ts = [T(mt, p) for p in parts]
    y = mt.concatenate(ts, dim=1)
    close(y.numpy(), np.concatenate(parts, axis=1))
    g = r.standard_normal(y.shape).astype(np.float32)
    y.backward(mt.DeviceArray.from_numpy(g))
    for t, piece in zip(ts, np.split(g, [3, 4], axis=1)):
        close(t.grad.numpy(), piece)
    same = [r.standard_normal((2, 3)).astype(np.float32) for _ in range(4)]
    for dim in (0, 1, -1):
        ts = [T(mt, p) for p in same]
        y = mt.stack(ts, dim=dim)
        close(y.numpy(), np.stack(same, axis=dim))
        g = r.standard_normal(y.shape).astype(np.float32)
        y.backward(mt.DeviceArray.from_numpy(g))
        for i, t in enumerate(ts):
            close(t.grad.numpy(), np.take(g, i, axis=dim))


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("float16", 1e-2)])
def test_reference_nonfused_attention_branch_runs_and_matches_fused(mt, dtype, tol):
    """gpt2_trainer/gpt2.py:168-203 on this package's Tensor: the qkv projection reshaped to
    [B,T,H,3D], transposed, chunked; scores with the additive causal mask buffer sliced to the
    sequence; softmax; @ v; merged back to [B,T,E] — equal to F.qkv_attention and to the oracle,
    forward and gradient."""
    Fn = mt.nn.functional
    r = np.random.default_rng(7)
    B, S, H, D, MAXS = 2, 48, 3, 32, 64
    E = H * D
    qkv = r.standard_normal((B, S, 3 * E)).astype(np.float32)
    do = r.standard_normal((B, S, E)).astype(np.float32)
    if dtype == "float16":
        qkv, do = qkv.astype(np.float16).astype(np.float32), do.astype(np.float16).astype(np.float32)
    mask = np.triu(np.full((MAXS, MAXS), -np.inf, np.float32), 1)[None, None]
    causal_mask = mt.Tensor(mask)                                   # the module's registered buffer

    x = mt.Tensor(mt.DeviceArray.from_numpy(qkv, dtype), requires_grad=True)
    t = x.reshape(B, S, H, 3 * D).transpose(1, 2)
    q, k, v = mt.chunk(t, 3, dim=-1)
    scores = (q @ k.transpose(-2, -1)) / (D ** 0.5)
    scores = scores + causal_mask[:, :, :S, :S].astype(scores.dtype)
    p = Fn.softmax(scores, dim=-1)
    out = (p @ v).transpose(1, 2).reshape(B, S, E)
    out.backward(mt.DeviceArray.from_numpy(do, dtype))

    x2 = mt.Tensor(mt.DeviceArray.from_numpy(qkv, dtype), requires_grad=True)
    fused = Fn.qkv_attention(x2, H, is_causal=True)
    fused.backward(mt.DeviceArray.from_numpy(do, dtype))

    q4 = qkv.reshape(B, S, H, 3 * D).transpose(0, 2, 1, 3)
    qn, kn, vn = (np.ascontiguousarray(q4[..., i * D:(i + 1) * D]) for i in range(3))
    o, pr = O.attention_fwd(qn, kn, vn, causal=True)
    dq, dk, dv = O.attention_bwd(qn, kn, vn, pr, do.reshape(B, S, H, D).transpose(0, 2, 1, 3))
    want_o = o.transpose(0, 2, 1, 3).reshape(B, S, E)
    want_g = np.concatenate([a.transpose(0, 2, 1, 3) for a in (dq, dk, dv)], axis=-1).reshape(B, S, 3 * E)
    close(out.numpy(), want_o, tol, "composed o"); close(fused.numpy(), want_o, tol, "fused o")
    close(x.grad.numpy(), want_g, 2 * tol, "composed dqkv"); close(x2.grad.numpy(), want_g, 2 * tol, "fused dqkv")
