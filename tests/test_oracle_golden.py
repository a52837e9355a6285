"""Pins the NumPy oracle against vectors produced by the unmodified reference
(tests/golden/generate.py). fp32 tolerance: 1e-4 relative to the tensor's max
magnitude (the tolerance the path's fp32 parity is stated at); most cases agree
to ~1e-6."""
import json
import os

import numpy as np
import pytest

from oracle import ops, gpt2 as og

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def close(a, b, rel=1e-4):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    scale = max(np.abs(b).max(), 1e-30)
    err = np.abs(a - b).max() / scale
    assert err <= rel, f"max err {err:.3e} of scale {scale:.3e}"


def test_layernorm(golden_ops, op_inputs):
    d, g = op_inputs, golden_ops
    y, mu, rs = ops.layernorm_fwd(d["ln_x"], d["ln_g"], d["ln_b"])
    dx, dg, db = ops.layernorm_bwd(d["ln_x"], mu, rs, d["ln_dy"], d["ln_g"])
    close(y, g["ln_y"]); close(dx, g["ln_dx"]); close(dg, g["ln_dg"]); close(db, g["ln_db"])
    y, mu, rs = ops.layernorm_fwd(d["ln_x"], d["ln_g"], None)
    dx, dg, _ = ops.layernorm_bwd(d["ln_x"], mu, rs, d["ln_dy"], d["ln_g"])
    close(y, g["ln_nb_y"]); close(dx, g["ln_nb_dx"]); close(dg, g["ln_nb_dg"])


def test_rmsnorm(golden_ops, op_inputs):
    d, g = op_inputs, golden_ops
    y, rs = ops.rmsnorm_fwd(d["rms_x"], d["rms_g"])
    dx, dg = ops.rmsnorm_bwd(d["rms_x"], rs, d["rms_dy"], d["rms_g"])
    close(y, g["rms_y"]); close(dx, g["rms_dx"]); close(dg, g["rms_dg"])
    y, rs = ops.rmsnorm_fwd(d["rms_x"], None)
    dx, _ = ops.rmsnorm_bwd(d["rms_x"], rs, d["rms_dy"], None)
    close(y, g["rms_nw_y"]); close(dx, g["rms_nw_dx"])


def test_softmax(golden_ops, op_inputs):
    d, g = op_inputs, golden_ops
    s = ops.softmax_fwd(d["sm_x"])
    close(s, g["sm_y"]); close(ops.softmax_bwd(d["sm_dy"], s), g["sm_dx"])


def test_linear(golden_ops, op_inputs):
    d, g = op_inputs, golden_ops
    close(ops.linear_fwd(d["lin_x"], d["lin_w"], d["lin_b"]), g["lin_y"])
    dx, dw, db = ops.linear_bwd(d["lin_x"], d["lin_w"], d["lin_dy"], True)
    close(dx, g["lin_dx"]); close(dw, g["lin_dw"]); close(db, g["lin_db"])


def test_activations(golden_ops, op_inputs):
    d, g = op_inputs, golden_ops
    close(ops.gelu_fwd(d["act_x"]), g["gelu_y"])
    close(ops.gelu_bwd(d["act_x"], d["act_dy"]), g["gelu_dx"])
    close(ops.relu2_fwd(d["act_x"]), g["relu2_y"])
    close(ops.relu2_bwd(d["act_x"], d["act_dy"]), g["relu2_dx"])


def test_cross_entropy(golden_ops, op_inputs):
    d, g = op_inputs, golden_ops
    close(ops.cross_entropy_fwd(d["ce_x"], d["ce_y"]), g["ce_loss"])
    close(ops.cross_entropy_bwd(d["ce_x"], d["ce_y"]), g["ce_dx"])
    loss, lse = ops.cross_entropy_rows(d["ce_x"], d["ce_y"])
    assert loss[3] == 0 and loss[17] == 0
    close(loss.sum() / 39, g["ce_loss"])


def test_embedding(golden_ops, op_inputs):
    d, g = op_inputs, golden_ops
    close(ops.embedding_fwd(d["emb_w"], d["emb_idx"]), g["emb_y"])
    close(ops.embedding_bwd(d["emb_dy"], d["emb_idx"], 23), g["emb_dw"])


def test_attention(golden_ops, op_inputs):
    d, g = op_inputs, golden_ops
    o, p = ops.attention_fwd(d["at_q"], d["at_k"], d["at_v"])
    dq, dk, dv = ops.attention_bwd(d["at_q"], d["at_k"], d["at_v"], p, d["at_do"])
    close(o, g["at_o"]); close(dq, g["at_dq"]); close(dk, g["at_dk"]); close(dv, g["at_dv"])


def test_rope(golden_ops, op_inputs):
    d, g = op_inputs, golden_ops
    cos, sin = ops.rope_cos_sin(32, 19)
    close(cos, g["rope_cos"]); close(sin, g["rope_sin"])
    close(ops.rope_fwd(d["rope_x"], cos, sin), g["rope_y"])
    close(ops.rope_bwd(d["rope_dy"], cos, sin), g["rope_dx"])


def test_adamw(golden_ops, op_inputs):
    d, g = op_inputs, golden_ops
    p = d["adam_p"].copy()
    m = np.zeros_like(p); v = np.zeros_like(p)
    b1p = b2p = 1.0
    for i in range(3):
        b1p *= 0.9; b2p *= 0.95
        ops.adamw_step(p, d["adam_g"][i], m, v, 3e-3, 0.9, 0.95, 1e-8, 0.1, b1p, b2p)
        close(p, g["adam_p"][i], rel=1e-6)
    close(m, g["adam_m"], rel=1e-6); close(v, g["adam_v"], rel=1e-6)


def test_grad_scaler_state_machine():
    s = ops.GradScaler(init_scale=8.0, growth_interval=3)
    s.update(True); assert s.scale == 4.0 and s.unskipped == 0
    s.update(False); s.update(False); assert s.scale == 4.0
    s.update(False); assert s.scale == 8.0 and s.unskipped == 0


def test_clip_grad_norm():
    g = [np.full(4, 3.0, np.float32), np.full(9, 4.0, np.float32)]
    n = ops.clip_grad_norm(g, 1.0)
    assert abs(n - np.sqrt(36 + 144)) < 1e-5
    assert abs(np.sqrt(sum((x ** 2).sum() for x in g)) - 1.0) < 1e-4


@pytest.fixture(scope="module")
def tiny_golden():
    with open(os.path.join(GOLDEN, "tiny_gpt2_fp32.json")) as fh:
        return json.load(fh)


def test_tiny_gpt2_first_step_matches_reference(tiny_golden):
    """Loss and every gradient norm of step 0, plus whole gradients of five
    tensors, against the reference run."""
    cfg = og.GPT2Config(65, 256, 256, 4, 4, 4)
    params = og.init_params(cfg, seed=0)
    x, y = og.synthetic_batch(np.random.default_rng(0), 16, 256, 65)
    loss, _, cache = og.forward(params, cfg, x, y)
    assert abs(float(loss) - tiny_golden["losses"][0]) <= 1e-5 * tiny_golden["losses"][0]
    grads = og.backward(params, cfg, cache)
    for k, ref in tiny_golden["first_step_grad_l2"].items():
        if k == "lm_head.weight":
            k = "embeddings.char_embeddings.weight"
        got = float(np.sqrt(np.sum(grads[k].astype(np.float64) ** 2)))
        assert abs(got - ref) <= 1e-4 * ref, (k, got, ref)
    whole = np.load(os.path.join(GOLDEN, "tiny_gpt2_first_grads.npz"))
    for k in whole.files:
        close(grads[k], whole[k])


def test_tiny_gpt2_loss_trajectory(tiny_golden):
    """First 8 optimizer steps of the 50-step reference run (the GPU test
    covers all 50; this keeps the CPU suite short)."""
    cfg = og.GPT2Config(65, 256, 256, 4, 4, 4)
    params = og.init_params(cfg, seed=0)
    losses = og.train(params, cfg, 8, 16, 256, data_seed=0)
    ref = tiny_golden["losses"][:8]
    for a, b in zip(losses, ref):
        assert abs(a - b) <= 1e-4 * abs(b), (losses, ref)


@pytest.mark.parametrize("fname,heads,seed", [("nanochat_tiny.json", dict(num_heads=2), 4),
                                              ("nanochat_tiny_gqa.json", dict(num_heads=4, num_kv_heads=2), 5)])
def test_nanochat_tiny_matches_reference(fname, heads, seed):
    """nanochat-style GPT oracle against the reference run (6 AdamW steps), multi-head and
    grouped-query (4 query heads on 2 key/value heads)."""
    from oracle import nanochat as on
    with open(os.path.join(GOLDEN, fname)) as fh:
        gold = json.load(fh)
    cfg = on.GPTConfig(vocab_size=96, max_seq_len=32, embed_dim=64, mlp_ratio=4, num_blocks=2, **heads)
    params = on.init_params(cfg, seed=seed)
    m = {k: np.zeros_like(v) for k, v in params.items()}
    v = {k: np.zeros_like(p) for k, p in params.items()}
    rng = np.random.default_rng(8)
    b1p = b2p = 1.0
    for step in range(6):
        x, y = og.synthetic_batch(rng, 3, 32, 96)
        loss, cache = on.forward(params, cfg, x, y)
        assert abs(float(loss) - gold["losses"][step]) <= 1e-4 * gold["losses"][step], (step, float(loss))
        grads = on.backward(params, cfg, cache)
        if step == 0:
            for k, ref in gold["first_step_grad_l2"].items():
                got = float(np.sqrt(np.sum(grads[k].astype(np.float64) ** 2)))
                assert abs(got - ref) <= 1e-4 * ref, (k, got, ref)
        b1p *= 0.9; b2p *= 0.95
        for k in params:
            ops.adamw_step(params[k], grads[k], m[k], v[k], 1e-3, 0.9, 0.95, 1e-8, 0.1, b1p, b2p)
