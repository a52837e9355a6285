"""End-to-end parity of the training step on the GPU: model + loss + backward +
AdamW through the public Python interface (which calls the C ABI), against the
reference's own loss trajectory (tests/golden/tiny_gpt2_fp32.json, produced by
the unmodified reference) and against the NumPy oracle."""
import json
import os

import numpy as np
import pytest

from oracle import gpt2 as og
from oracle import ops as O

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def build(cfg, params, dtype="float32"):
    import mytorch_b200 as mt
    from mytorch_b200.gpt2 import GPT2, GPT2Config
    np.random.seed(0)
    model = GPT2(GPT2Config(vocab_size=cfg.vocab_size, max_seq_len=cfg.max_seq_len, embed_dim=cfg.embed_dim,
                            mlp_ratio=cfg.mlp_ratio, num_blocks=cfg.num_blocks, num_heads=cfg.num_heads))
    sd = dict(params)
    sd["lm_head.weight"] = params["embeddings.char_embeddings.weight"]
    model.load_state_dict(sd)
    return mt, model


def groups(model, wd=0.1):
    decay, no_decay = [], []
    for _, p in model.named_parameters():
        (no_decay if len(p.shape) < 2 else decay).append(p)
    return [{"params": decay, "weight_decay": wd}, {"params": no_decay, "weight_decay": 0.0}]


def test_tiny_gpt2_fp32_50_steps_match_reference_losses():
    """Config: L4 H4 d256 ctx256 vocab65 batch16, AdamW lr3e-4 betas(0.9,0.95)
    wd0.1, seed-0 token ids; the first 50 losses must be within 1e-3 relative
    of the reference fp32 run."""
    with open(os.path.join(GOLDEN, "tiny_gpt2_fp32.json")) as fh:
        gold = json.load(fh)
    cfg = og.GPT2Config(65, 256, 256, 4, 4, 4)
    mt, model = build(cfg, og.init_params(cfg, seed=0))
    opt = mt.optim.AdamW(groups(model), lr=3e-4, beta1=0.9, beta2=0.95)
    loss_fn = mt.nn.CrossEntropyLoss()
    rng = np.random.default_rng(0)
    losses = []
    for step in range(50):
        x, y = og.synthetic_batch(rng, 16, 256, 65)
        logits = model(mt.Tensor(x))
        loss = loss_fn(logits, mt.Tensor(y))
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    ref = np.array(gold["losses"])
    rel = np.abs(np.array(losses) - ref) / np.abs(ref)
    assert rel.max() <= 1e-3, (rel.max(), losses[:5], ref[:5])
    final = model.state_dict()
    for k, want in gold["final_weight_l2"].items():
        got = float(np.sqrt(np.sum(final[k].astype(np.float64) ** 2)))
        assert abs(got - want) <= 1e-3 * want, (k, got, want)


def test_backward_timing_table(capsys):
    """loss.backward(time_backward=True) reports the device time of every backward closure by name
    (mytorch/tensor.py:221-261) and leaves the gradients unchanged."""
    cfg = og.GPT2Config(65, 64, 64, 4, 2, 2)
    params = og.init_params(cfg, seed=0)
    x, y = og.synthetic_batch(np.random.default_rng(0), 4, 64, 65)
    grads = []
    for timed in (False, True):
        mt, model = build(cfg, params)
        loss = mt.nn.CrossEntropyLoss()(model(mt.Tensor(x)), mt.Tensor(y))
        loss.backward(time_backward=timed, num_ops_to_show=5)
        grads.append({n: p.grad.numpy() for n, p in model.named_parameters()})
    out = capsys.readouterr().out
    assert "most time-consuming backward functions" in out and "<LinearBackward>" in out
    table = mt.Tensor.last_backward_timings
    assert table["<MLPBackward>"][1] == 2 and all(ms >= 0 for ms, _ in table.values())
    for k in grads[0]:
        assert np.array_equal(grads[0][k], grads[1][k]) or np.allclose(grads[0][k], grads[1][k], rtol=1e-5, atol=1e-7), k


def test_first_step_gradients_match_reference():
    cfg = og.GPT2Config(65, 256, 256, 4, 4, 4)
    mt, model = build(cfg, og.init_params(cfg, seed=0))
    x, y = og.synthetic_batch(np.random.default_rng(0), 16, 256, 65)
    loss = mt.nn.CrossEntropyLoss()(model(mt.Tensor(x)), mt.Tensor(y))
    loss.backward()
    whole = np.load(os.path.join(GOLDEN, "tiny_gpt2_first_grads.npz"))
    grads = {n: p.grad.numpy() for n, p in model.named_parameters()}
    for k in whole.files:
        want = whole[k]
        err = np.abs(grads[k] - want).max() / np.abs(want).max()
        assert err <= 1e-4, (k, err)


@pytest.mark.parametrize("half", ["float16", "bfloat16"])
def test_mixed_precision_step_tracks_fp32_oracle(half):
    """Small GPT-2 under the Accelerator (half activations, fp32 masters, loss
    scaling, accumulation 2, clip 1.0): losses stay within 1e-2 of the fp32
    oracle driven with the same batches, and the weights move the same way."""
    cfg = og.GPT2Config(vocab_size=264, max_seq_len=64, embed_dim=128, mlp_ratio=4, num_blocks=2, num_heads=2)
    params = og.init_params(cfg, seed=3)
    mt, model = build(cfg, params)
    acc = mt.Accelerator(num_gpus=1, rank=0, gradient_accumulation_steps=2, mixed_precision=True, half_dtype=half)
    opt = mt.optim.AdamW(groups(model), lr=1e-3, beta1=0.9, beta2=0.95)
    model, opt = acc.prepare(model, opt)
    loss_fn = mt.nn.CrossEntropyLoss()
    ref_params = {k: v.copy() for k, v in params.items()}
    ref_opt = og.AdamW(ref_params, 1e-3, 0.9, 0.95, 1e-8, 0.1)
    rng = np.random.default_rng(5)
    got, want = [], []
    for step in range(6):
        gsum = None
        for micro in range(2):
            x, y = og.synthetic_batch(rng, 4, 64, 264)
            loss = loss_fn(model(mt.Tensor(x)), mt.Tensor(y))
            acc.backward(loss)
            acc.clip_grad_norm_(1.0)
            opt.step()
            opt.zero_grad()
            got.append(loss.item())
            rl, _, cache = og.forward(ref_params, cfg, x, y)
            g = og.backward(ref_params, cfg, cache)
            gsum = g if gsum is None else {k: gsum[k] + g[k] for k in g}
            want.append(float(rl))
        gsum = {k: v / 2 for k, v in gsum.items()}
        O.clip_grad_norm(list(gsum.values()), 1.0)
        ref_opt.step(ref_params, gsum)
    got, want = np.array(got), np.array(want)
    assert np.abs(got - want).max() / want.max() <= 1e-2, (got, want)
    assert acc.scaler.skipped_steps == 0
    # masters follow the oracle's weights
    for name, p in model._named_parameters_no_dedup():
        i = acc._param_index[id(p)]
        m = acc._flat.view(acc._flat.master, i).numpy()
        ref = ref_params.get(name, ref_params["embeddings.char_embeddings.weight"])
        assert np.abs(m - ref).max() <= 6e-3 * max(1.0, np.abs(ref).max()), name   # 6 steps of lr 1e-3


def test_gpt2_124m_fp16_amp_steps_track_fp32_oracle():
    """The full GPT-2 124M (L12 H12 d768 ctx1024, vocabulary padded to 50304, tied head) under
    fp16 mixed precision with dynamic loss scaling, AdamW lr 6e-4 wd 0.1, clip 1.0, on one
    sequence of 1024 tokens: five steps on it, losses within 1e-2 of the fp32 oracle stepping the
    same weights on the same batch (the oracle needs a few seconds per step at this size)."""
    cfg = og.GPT2Config(vocab_size=50304, max_seq_len=1024, embed_dim=768, mlp_ratio=4, num_blocks=12, num_heads=12)
    params = og.init_params(cfg, seed=0)
    mt, model = build(cfg, params)
    acc = mt.Accelerator(num_gpus=1, rank=0, mixed_precision=True)
    opt = mt.optim.AdamW(groups(model), lr=6e-4, beta1=0.9, beta2=0.95)
    model, opt = acc.prepare(model, opt)
    loss_fn = mt.nn.CrossEntropyLoss(fused_backward=True)      # the loss path the benchmark uses
    ref_opt = og.AdamW(params, 6e-4, 0.9, 0.95, 1e-8, 0.1)
    x, y = og.synthetic_batch(np.random.default_rng(3), 1, 1024, 50257)    # one batch, revisited: the loss moves fast
    got, want = [], []
    for step in range(5):
        loss = loss_fn(model(mt.Tensor(x)), mt.Tensor(y))
        acc.backward(loss)
        acc.clip_grad_norm_(1.0)
        opt.step()
        opt.zero_grad()
        got.append(loss.item())
        rl, _, cache = og.forward(params, cfg, x, y)
        g = og.backward(params, cfg, cache)
        O.clip_grad_norm(list(g.values()), 1.0)
        ref_opt.step(params, g)
        want.append(float(rl))
    got, want = np.array(got), np.array(want)
    assert acc.scaler.skipped_steps == 0
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max(), (got, want)
    assert want.min() < want[0] - 0.5, want      # the steps did move the loss, so the comparison means something


def test_overflow_skips_the_step_and_halves_the_scale():
    """An inf planted in the gradient buffer (host-made input, no device fault):
    the fused update must leave weights and moments untouched, clear nothing it
    should not, and the device-side scaler must back off."""
    cfg = og.GPT2Config(vocab_size=64, max_seq_len=32, embed_dim=64, mlp_ratio=4, num_blocks=1, num_heads=2)
    mt, model = build(cfg, og.init_params(cfg, seed=1))
    acc = mt.Accelerator(num_gpus=1, rank=0, mixed_precision=True)
    opt = mt.optim.AdamW(groups(model), lr=1e-3)
    model, opt = acc.prepare(model, opt)
    before = acc._flat.master.numpy().copy()
    x, y = og.synthetic_batch(np.random.default_rng(0), 2, 32, 64)
    loss = mt.nn.CrossEntropyLoss()(model(mt.Tensor(x)), mt.Tensor(y))
    acc.step_counter = 0
    loss.backward(acc.scaler.scale_dev)
    g = acc._flat.grad.numpy()
    g[5] = np.inf
    acc._flat.grad.set_from_numpy(g)
    acc.step_counter = 1
    acc._grads_ready = False
    acc.clip_grad_norm_(1.0)
    opt.step()
    opt.zero_grad()
    assert acc.scaler.scale == 2.0 ** 15 and acc.scaler.skipped_steps == 1
    assert np.array_equal(acc._flat.master.numpy(), before)
    assert not acc._flat.m.numpy().any()
    assert not acc._flat.grad.numpy().any()
    # the skipped step advanced neither the step count nor the beta powers (the reference does not
    # call optimizer.step() on an overflow, mytorch/accelerate.py:342-352)
    for st in opt.state_dict()["state"]:
        assert (st["t"], st["beta1_pow"], st["beta2_pow"]) == (0, 1.0, 1.0), st
    # the next clean step proceeds, with the bias correction of a FIRST step
    loss = mt.nn.CrossEntropyLoss()(model(mt.Tensor(x)), mt.Tensor(y))
    acc.backward(loss)
    opt.step()
    assert not np.array_equal(acc._flat.master.numpy(), before)
    assert acc.scaler.unskipped == 1
    for st, grp in zip(opt.state_dict()["state"], opt.param_groups):
        assert st["t"] == 1 and st["beta1_pow"] == grp["beta1"] and st["beta2_pow"] == grp["beta2"], st


def test_adamw_multi_tensor_matches_reference_golden(golden_ops, op_inputs):
    import mytorch_b200 as mt
    d, g = op_inputs, golden_ops
    p = mt.Tensor(d["adam_p"].copy(), requires_grad=True)
    p.is_param = True
    opt = mt.optim.AdamW([{"params": [p], "weight_decay": 0.1}], lr=3e-3, beta1=0.9, beta2=0.95)
    for i in range(3):
        p.grad = mt.DeviceArray.from_numpy(d["adam_g"][i])
        opt.step()
        assert np.abs(p.numpy() - g["adam_p"][i]).max() <= 1e-6 * np.abs(g["adam_p"][i]).max() + 1e-7
    assert np.abs(opt.param_groups[0]["m"][0].numpy() - g["adam_m"]).max() <= 1e-6
    assert np.abs(opt.param_groups[0]["v"][0].numpy() - g["adam_v"]).max() <= 1e-6


@pytest.mark.parametrize("fname,hq,hkv,seed", [("nanochat_tiny.json", 2, 2, 4), ("nanochat_tiny_gqa.json", 4, 2, 5)])
def test_nanochat_tiny_fp32_matches_reference_losses(fname, hq, hkv, seed):
    """nanochat-style GPT (RoPE then QK-norm, parameter-free RMSNorm, ReLU^2,
    untied head, soft-capped loss) through the CUDA library against the
    reference runs in tests/golden/: multi-head, and grouped-query with 4 query heads on 2
    key/value heads."""
    import mytorch_b200 as mt
    from mytorch_b200.nanochat_gpt import GPT, GPTConfig
    from oracle import nanochat as on
    with open(os.path.join(GOLDEN, fname)) as fh:
        gold = json.load(fh)
    cfg = on.GPTConfig(vocab_size=96, max_seq_len=32, embed_dim=64, mlp_ratio=4, num_blocks=2, num_heads=hq,
                       num_kv_heads=hkv)
    np.random.seed(0)
    model = GPT(GPTConfig(vocab_size=96, max_seq_len=32, embed_dim=64, mlp_ratio=4, num_blocks=2,
                          num_q_heads=hq, num_kv_heads=hkv))
    model.load_state_dict(on.init_params(cfg, seed=seed))
    opt = mt.optim.AdamW([{"params": model.parameters(), "weight_decay": 0.1}], lr=1e-3, beta1=0.9, beta2=0.95)
    rng = np.random.default_rng(8)
    for step in range(6):
        x, y = og.synthetic_batch(rng, 3, 32, 96)
        _, loss = model(mt.Tensor(x), mt.Tensor(y))
        loss.backward()
        if step == 0:
            for n, p in model.named_parameters():
                got = float(np.sqrt(np.sum(p.grad.numpy().astype(np.float64) ** 2)))
                ref = gold["first_step_grad_l2"][n]
                assert abs(got - ref) <= 1e-4 * ref, (n, got, ref)
        opt.step()
        opt.zero_grad()
        assert abs(loss.item() - gold["losses"][step]) <= 1e-3 * gold["losses"][step], (step, loss.item())
    final = model.state_dict()
    for k, want in gold["final_weight_l2"].items():
        got = float(np.sqrt(np.sum(final[k].astype(np.float64) ** 2)))
        assert abs(got - want) <= 1e-3 * want, (k, got, want)


def test_nanochat_half_precision_head_dim_128_runs_on_tensor_cores():
    """bf16 step of a small nanochat model with head_dim 128 (the d20 head size):
    loss within 2e-2 of the fp32 oracle on the same weights and batch."""
    import mytorch_b200 as mt
    from mytorch_b200.nanochat_gpt import GPT, GPTConfig
    from oracle import nanochat as on
    cfg = on.GPTConfig(vocab_size=512, max_seq_len=256, embed_dim=256, mlp_ratio=4, num_blocks=2, num_heads=2)
    params = on.init_params(cfg, seed=6)
    np.random.seed(0)
    model = GPT(GPTConfig(vocab_size=512, max_seq_len=256, embed_dim=256, mlp_ratio=4, num_blocks=2,
                          num_q_heads=2, num_kv_heads=2))
    model.load_state_dict(params)
    acc = mt.Accelerator(num_gpus=1, rank=0, mixed_precision=True, half_dtype="bfloat16")
    opt = mt.optim.AdamW([{"params": model.parameters(), "weight_decay": 0.0}], lr=1e-3)
    model, opt = acc.prepare(model, opt)
    x, y = og.synthetic_batch(np.random.default_rng(2), 2, 256, 512)
    _, loss = model(mt.Tensor(x), mt.Tensor(y))
    acc.backward(loss)
    opt.step()
    want, _ = on.forward(params, cfg, x, y)
    assert abs(loss.item() - float(want)) <= 2e-2 * float(want), (loss.item(), float(want))
    assert acc.scaler.skipped_steps == 0
    import ctypes
    f = ctypes.c_int(0)
    mt._lib.device_flag_read(ctypes.byref(f), mt.stream())
    assert f.value == 0


def test_nanochat_d20_width_fp16_steps_track_fp32_oracle():
    """A two-block stack at the d20 model's width (d1280, 10 heads of 128, vocabulary 65536,
    ReLU^2 MLP of 5120, rotary + QK-norm, soft-capped loss) in fp16 mixed precision: three AdamW
    steps on one batch, losses within 1e-2 of the fp32 oracle stepping the same weights; and the
    three ways the model can produce its loss agree on the first step."""
    import mytorch_b200 as mt
    from mytorch_b200.nanochat_gpt import GPT, GPTConfig
    from oracle import nanochat as on
    cfg = on.GPTConfig(vocab_size=65536, max_seq_len=256, embed_dim=1280, mlp_ratio=4, num_blocks=2, num_heads=10)
    params = on.init_params(cfg, seed=2)
    params["embeddings.embeddings.weight"] *= 0.04      # token embeddings at the model's own scale (std 0.02)
    x, y = og.synthetic_batch(np.random.default_rng(4), 2, 256, 65536)

    def make(mode):
        np.random.seed(0)
        model = GPT(GPTConfig(vocab_size=65536, max_seq_len=256, embed_dim=1280, mlp_ratio=4, num_blocks=2,
                              num_q_heads=10, num_kv_heads=10))
        model.load_state_dict(params)
        model.loss_mode = mode
        acc = mt.Accelerator(num_gpus=1, rank=0, mixed_precision=True)
        opt = mt.optim.AdamW([{"params": model.parameters(), "weight_decay": 0.1}], lr=3e-4, beta1=0.9, beta2=0.95)
        model, opt = acc.prepare(model, opt)
        return model, acc, opt

    first = {}
    for mode in ("logits", "chunked"):
        model, acc, opt = make(mode)
        _, loss = model(mt.Tensor(x), mt.Tensor(y))
        first[mode] = loss.item()
        del model, acc, opt
    model, acc, opt = make("fused")
    ref_opt = og.AdamW(params, 3e-4, 0.9, 0.95, 1e-8, 0.1)
    got, want = [], []
    for step in range(3):
        logits, loss = model(mt.Tensor(x), mt.Tensor(y))
        assert logits is None
        acc.backward(loss)
        acc.clip_grad_norm_(1.0)
        opt.step()
        opt.zero_grad()
        got.append(loss.item())
        rl, cache = on.forward(params, cfg, x, y)
        g = on.backward(params, cfg, cache)
        O.clip_grad_norm(list(g.values()), 1.0)
        ref_opt.step(params, g)
        want.append(float(rl))
    got, want = np.array(got), np.array(want)
    assert acc.scaler.skipped_steps == 0
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max(), (got, want)
    for mode, v in first.items():
        assert abs(v - want[0]) <= 1e-2 * want[0], (mode, v, want[0])
    import ctypes
    f = ctypes.c_int(0)
    mt._lib.device_flag_read(ctypes.byref(f), mt.stream())
    assert f.value == 0


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("float16", 1e-2)])
@pytest.mark.parametrize("softcap", [None, 15.0])
def test_chunked_lm_head_cross_entropy_matches_unfused(dtype, tol, softcap):
    """F.lm_head_cross_entropy (vocabulary in chunks, logits never materialised)
    against linear + cross_entropy of the same library and against the oracle,
    loss and both gradients; vocab 1000 in chunks of 256 (ragged last chunk)."""
    import mytorch_b200 as mt
    F = mt.nn.functional
    r = np.random.default_rng(21)
    M, E, V = 192, 64, 1000
    x = r.standard_normal((M, E)).astype(np.float32)
    w = (r.standard_normal((V, E)) * 0.3).astype(np.float32)
    y = r.integers(0, V, M).astype(np.int32)
    y[5] = -100
    if dtype == "float16":
        x, w = x.astype(np.float16).astype(np.float32), w.astype(np.float16).astype(np.float32)

    def run(fused):
        X = mt.Tensor(mt.DeviceArray.from_numpy(x, dtype), requires_grad=True)
        W = mt.nn.Parameter(mt.DeviceArray.from_numpy(w, dtype))
        Y = mt.Tensor(y)
        loss = (F.lm_head_cross_entropy(X, W, Y, chunk=256, softcap=softcap) if fused
                else F.cross_entropy(F.linear(X, W), Y, softcap=softcap))
        loss.backward()
        return loss.item(), X.grad.numpy().astype(np.float64), W.grad.numpy().astype(np.float64)

    lf, dxf, dwf = run(True)
    lu, dxu, dwu = run(False)
    logits = x @ w.T
    if softcap:
        t = np.tanh(logits / softcap)
        want = float(O.cross_entropy_fwd(softcap * t, y))
        dl = O.cross_entropy_bwd(softcap * t, y) * (1 - t * t)
    else:
        want = float(O.cross_entropy_fwd(logits, y))
        dl = O.cross_entropy_bwd(logits, y)
    for name, got, ref in (("loss", lf, want), ("loss unfused", lu, want)):
        assert abs(got - ref) <= tol * abs(ref), (name, got, ref)
    for name, got, ref in (("dx", dxf, dl @ w), ("dw", dwf, dl.T @ x), ("dx unfused", dxu, dl @ w), ("dw unfused", dwu, dl.T @ x)):
        err = np.abs(got - ref).max() / np.abs(ref).max()
        assert err <= 2 * tol, (name, err)


def test_checkpoint_files_match_reference_layout_and_resume(tmp_path):
    """save_state writes the reference's three files (accelerate.py:916-975): model.safetensors
    with the fp32 masters, optimizer.bin = pickled AdamW.state_dict() in the layout of
    optimizers.py:378-407, mp_config.bin with the scaler fields; a fresh process-equivalent
    (new model, optimizer, Accelerator) that loads them continues on the same losses."""
    import pickle
    from safetensors.numpy import load_file
    cfg = og.GPT2Config(vocab_size=264, max_seq_len=64, embed_dim=128, mlp_ratio=4, num_blocks=2, num_heads=2)
    params = og.init_params(cfg, seed=6)

    def make():
        mt, model = build(cfg, {k: v.copy() for k, v in params.items()})
        acc = mt.Accelerator(num_gpus=1, rank=0, mixed_precision=True)
        opt = mt.optim.AdamW(groups(model), lr=1e-3, beta1=0.9, beta2=0.95)
        model, opt = acc.prepare(model, opt)
        return mt, model, acc, opt

    def run(mt, model, acc, opt, rng, steps):
        out = []
        for _ in range(steps):
            x, y = og.synthetic_batch(rng, 4, 64, 264)
            loss = mt.nn.CrossEntropyLoss()(model(mt.Tensor(x)), mt.Tensor(y))
            acc.backward(loss)
            acc.clip_grad_norm_(1.0)
            opt.step()
            opt.zero_grad()
            out.append(loss.item())
        return out

    rng = np.random.default_rng(9)
    mt, model, acc, opt = make()
    run(mt, model, acc, opt, rng, 3)
    ckpt = str(tmp_path / "ckpt")
    acc.save_state(ckpt)
    rng_state = rng.bit_generator.state
    straight = run(mt, model, acc, opt, rng, 3)

    weights = load_file(ckpt + "/model.safetensors")
    names = [n for n, _ in model._named_parameters_no_dedup()]
    assert sorted(weights) == sorted(names) and all(w.dtype == np.float32 for w in weights.values())
    with open(ckpt + "/optimizer.bin", "rb") as fh:
        osd = pickle.load(fh)
    assert set(osd) == {"state", "param_groups"} and len(osd["state"]) == 2
    assert set(osd["state"][0]) == {"m", "v", "t", "beta1_pow", "beta2_pow"} and osd["state"][0]["t"] == 3
    assert set(osd["param_groups"][0]) == {"lr", "beta1", "beta2", "eps", "weight_decay", "num_params"}
    with open(ckpt + "/mp_config.bin", "rb") as fh:
        assert set(pickle.load(fh)) == {"scale", "growth_factor", "backoff_factor", "growth_interval", "unskipped"}

    mt2, model2, acc2, opt2 = make()
    acc2.load_state(ckpt)
    rng2 = np.random.default_rng(0)
    rng2.bit_generator.state = rng_state
    resumed = run(mt2, model2, acc2, opt2, rng2, 3)
    # split-K gradient accumulation adds in a scheduling-dependent order: equal to fp32 round-off
    assert np.allclose(resumed, straight, rtol=2e-4, atol=0), (resumed, straight)


def test_checkpoint_carries_the_prepared_dataloader(tmp_path):
    """A loader handed to Accelerator.prepare is written as dataloader_0.bin (accelerate.py:970-976)
    and a resumed run continues on the batch after the last one consumed, in the same shuffled
    order; a checkpoint without the file warns and starts the epoch over (accelerate.py:1036-1047)."""
    import os
    import pickle
    import warnings
    import mytorch_b200 as mt
    from mytorch_b200.utils.data import DataLoader, Dataset

    class Rows(Dataset):
        def __len__(self):
            return 37

        def __getitem__(self, i):
            return np.array([i, 2 * i], dtype=np.int32)

    np.random.seed(11)
    acc = mt.Accelerator(num_gpus=1, rank=0)
    (dl,) = acc.prepare(DataLoader(Rows(), batch_size=4, shuffle=True))
    it = iter(dl)
    seen = [next(it)[:, 0].copy() for _ in range(3)]
    ckpt = str(tmp_path / "ckpt")
    acc.save_state(ckpt)
    rest = []
    while True:
        try:
            rest.append(next(it)[:, 0].copy())
        except StopIteration:
            break
    with open(os.path.join(ckpt, "dataloader_0.bin"), "rb") as fh:
        st = pickle.load(fh)
    assert st["batches_consumed"] == 3 and st["epoch"] == 0 and len(st["shuffled_indices"]) == 37

    acc2 = mt.Accelerator(num_gpus=1, rank=0)
    (dl2,) = acc2.prepare(DataLoader(Rows(), batch_size=4, shuffle=True))
    acc2.load_state(ckpt)
    rest2 = [b[:, 0].copy() for b in dl2]
    assert len(rest2) == len(rest) and all(np.array_equal(a, b) for a, b in zip(rest, rest2))
    assert sorted(np.concatenate(seen + rest2).tolist()) == list(range(37))

    os.remove(os.path.join(ckpt, "dataloader_0.bin"))
    acc3 = mt.Accelerator(num_gpus=1, rank=0)
    acc3.prepare(DataLoader(Rows(), batch_size=4, shuffle=True))
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        acc3.load_state(ckpt)
    assert any("cannot resume dataloader" in str(x.message) for x in w)


def test_dataloader_device_staging_feeds_the_same_batches():
    """The staged host -> device path (pinned buffers, copy stream, uint16 widened on the device)
    hands out exactly the host batches, in order, across buffer reuse; a training loop fed by it
    reaches the losses of the same loop fed with host arrays."""
    import mytorch_b200 as mt
    from mytorch_b200.utils.data import DataLoader, TokenLoader
    toks = np.random.default_rng(2).integers(0, 264, 40000).astype(np.uint16)
    ds = TokenLoader(toks, 64, virtual_length=40, seed=7)
    host = [(x.copy(), y.copy()) for x, y in DataLoader(ds, batch_size=4, num_workers=2)]
    dev = []
    for x, y in DataLoader(ds, batch_size=4, num_workers=2, device=True, staging_depth=2):
        assert x.data.dtype == "int32" and x.shape == (4, 64)
        dev.append((x.numpy().copy(), y.numpy().copy()))
    assert len(dev) == len(host) == 10
    for (hx, hy), (dx, dy) in zip(host, dev):
        assert np.array_equal(hx.astype(np.int32), dx) and np.array_equal(hy.astype(np.int32), dy)

    cfg = og.GPT2Config(vocab_size=264, max_seq_len=64, embed_dim=128, mlp_ratio=4, num_blocks=2, num_heads=2)
    params = og.init_params(cfg, seed=8)

    def train(batches):
        mt_, model = build(cfg, {k: v.copy() for k, v in params.items()})
        opt = mt_.optim.AdamW(groups(model), lr=1e-3, beta1=0.9, beta2=0.95)
        losses = []
        for x, y in batches:
            x = x if isinstance(x, mt_.Tensor) else mt_.Tensor(x.astype(np.int32))
            y = y if isinstance(y, mt_.Tensor) else mt_.Tensor(y.astype(np.int32))
            loss = mt_.nn.CrossEntropyLoss()(model(x), y)
            loss.backward()
            opt.step()
            opt.zero_grad()
            losses.append(loss.item())
        return losses

    a = train(host[:6])
    b = train(DataLoader(TokenLoader(toks, 64, virtual_length=24, seed=7), batch_size=4, num_workers=2, device=True))
    assert np.allclose(a, b, rtol=1e-5), (a, b)


def test_gradient_checkpointing_gives_the_same_training_run():
    """Blocks recomputed in the backward pass (utils/checkpoint.py, gpt2.py:349-365): same losses
    and weights as the plain run (the recomputation repeats the same kernels on the same inputs)."""
    cfg = og.GPT2Config(vocab_size=264, max_seq_len=128, embed_dim=128, mlp_ratio=4, num_blocks=4, num_heads=2)
    params = og.init_params(cfg, seed=10)

    def train(ckpt):
        mt, model = build(cfg, {k: v.copy() for k, v in params.items()})
        if ckpt:
            model.enable_gradient_checkpointing()
        opt = mt.optim.AdamW(groups(model), lr=1e-3, beta1=0.9, beta2=0.95)
        rng = np.random.default_rng(11)
        losses = []
        for _ in range(3):
            x, y = og.synthetic_batch(rng, 8, 128, 264)
            loss = mt.nn.CrossEntropyLoss()(model(mt.Tensor(x)), mt.Tensor(y))
            loss.backward()
            opt.step()
            opt.zero_grad()
            losses.append(loss.item())
        return losses, model.state_dict()

    l0, w0 = train(False)
    l1, w1 = train(True)
    assert np.allclose(l0, l1, rtol=1e-6), (l0, l1)
    for k in w0:
        assert np.allclose(w0[k], w1[k], rtol=0, atol=1e-6), k


def test_kv_cache_decoding_matches_the_full_forward():
    """The inference step (gpt2.py:29-86, :167-215): prompt through the cache, then one token at
    a time; at every step the last-position logits equal those of the oracle's full forward over
    the whole prefix (fp32, 1e-4). Also two tokens in one step and greedy generate() with and
    without the cache."""
    import mytorch_b200 as mt
    from mytorch_b200.gpt2 import Cache
    cfg = og.GPT2Config(vocab_size=264, max_seq_len=64, embed_dim=128, mlp_ratio=4, num_blocks=2, num_heads=2)
    params = og.init_params(cfg, seed=12)
    _, model = build(cfg, params)
    model.eval()
    ids = np.random.default_rng(13).integers(0, 264, (3, 40)).astype(np.int32)
    cache = Cache(model.config)
    with mt.no_grad():
        logits, cache = model(mt.Tensor(ids[:, :17]), cache=cache)
        steps = [(17, logits.numpy()[:, -1])]
        for n in range(17, 30):
            logits, cache = model(mt.Tensor(ids[:, n:n + 1]), cache=cache)
            steps.append((n + 1, logits.numpy()[:, -1]))
        logits, cache = model(mt.Tensor(ids[:, 30:32]), cache=cache)     # two new tokens at once
        assert cache.get_seq_len() == 32 and logits.shape == (3, 2, 264)
    for n, got in steps:
        want = og.forward(params, cfg, ids[:, :n])[1].reshape(3, n, -1)[:, -1]
        assert np.abs(got.astype(np.float64) - want).max() <= 1e-4 * np.abs(want).max(), n
    a = model.generate(ids[:, :8], 6, temperature=0, use_cache=True)
    b = model.generate(ids[:, :8], 6, temperature=0, use_cache=False)
    assert a.shape == (3, 14) and np.array_equal(a, b)


def test_fused_cross_entropy_backward_trains_like_the_two_pass_form():
    """CrossEntropyLoss(fused_backward=True): the gradient is produced in the forward pass with the
    loss scale announced by the Accelerator folded in; plain loss.backward() (upstream 1) and a
    backward with an unannounced gradient (corrected by the extra pass) give the same results as
    the two-pass form."""
    import mytorch_b200 as mt
    cfg = og.GPT2Config(vocab_size=264, max_seq_len=64, embed_dim=128, mlp_ratio=4, num_blocks=2, num_heads=2)
    params = og.init_params(cfg, seed=14)

    def amp_run(fused):
        mt_, model = build(cfg, {k: v.copy() for k, v in params.items()})
        acc = mt_.Accelerator(num_gpus=1, rank=0, mixed_precision=True)
        opt = mt_.optim.AdamW(groups(model), lr=1e-3, beta1=0.9, beta2=0.95)
        model, opt = acc.prepare(model, opt)
        loss_fn = mt_.nn.CrossEntropyLoss(fused_backward=fused)
        rng = np.random.default_rng(15)
        out = []
        for _ in range(4):
            x, y = og.synthetic_batch(rng, 4, 64, 264)
            loss = loss_fn(model(mt_.Tensor(x)), mt_.Tensor(y))
            acc.backward(loss)
            acc.clip_grad_norm_(1.0)
            opt.step(); opt.zero_grad()
            out.append(loss.item())
        return out, acc._flat.master.numpy().copy()

    (la, wa), (lb, wb) = amp_run(False), amp_run(True)
    assert np.allclose(la, lb, rtol=2e-3), (la, lb)
    assert np.abs(wa - wb).max() <= 2e-3

    def fp32_grads(fused, upstream):
        mt.Tensor.loss_grad_hint = None
        mt_, model = build(cfg, {k: v.copy() for k, v in params.items()})
        x, y = og.synthetic_batch(np.random.default_rng(16), 4, 64, 264)
        loss = mt_.nn.CrossEntropyLoss(fused_backward=fused)(model(mt_.Tensor(x)), mt_.Tensor(y))
        if upstream is None:
            loss.backward()
        else:
            loss.backward(mt_.DeviceArray.from_numpy(np.array(upstream, np.float32)))
        return {n: p.grad.numpy().copy() for n, p in model.named_parameters()}

    for upstream in (None, 2.5):
        ga, gb = fp32_grads(False, upstream), fp32_grads(True, upstream)
        for n in ga:
            assert np.abs(ga[n] - gb[n]).max() <= 1e-5 * max(1.0, np.abs(ga[n]).max()), (n, upstream)


@pytest.mark.parametrize("kv_heads", [2, 1])
def test_nanochat_kv_cache_decoding_matches_the_full_forward(kv_heads):
    """nanochat inference branch (nanochat_gpt.py:301-340, core/cache.py): prompt then token by
    token through the KVCache (rotary positions continue after the cache, head_dim 128 through the
    decode-attention kernel) gives the soft-capped logits of the uncached forward, which the
    training parity test pins to the reference. With one key/value head for the two query heads
    the cache holds that one head and both query heads read it (grouped-query attention)."""
    import mytorch_b200 as mt
    from mytorch_b200.nanochat_gpt import GPT, GPTConfig, KVCache
    cfg = GPTConfig(vocab_size=160, max_seq_len=48, embed_dim=256, mlp_ratio=4, num_blocks=2, num_q_heads=2,
                    num_kv_heads=kv_heads)
    np.random.seed(5)
    model = GPT(cfg)
    r = np.random.default_rng(6)
    for n, p in model.named_parameters():          # out_proj / lm_head start at zero: give them values
        if "out_proj" in n or "lm_head" in n:
            p.data.set_from_numpy((r.standard_normal(p.shape) * 0.05).astype(np.float32))
    model.eval()
    ids = r.integers(0, 160, (2, 30)).astype(np.int32)
    with mt.no_grad():
        full = model(mt.Tensor(ids), None)[0].numpy()
        assert np.abs(full).max() <= cfg.softcap
        cache = KVCache(2, kv_heads, 48, 128, 2)
        out, cache = model(mt.Tensor(ids[:, :11]), None, cache=cache)
        got = [out.numpy()]
        for n in range(11, 26):
            out, cache = model(mt.Tensor(ids[:, n:n + 1]), None, cache=cache)
            got.append(out.numpy())
        out, cache = model(mt.Tensor(ids[:, 26:30]), None, cache=cache)   # four tokens in one step, causal among them
        got.append(out.numpy())
        assert cache.pos == 30
    got = np.concatenate(got, axis=1)
    assert np.abs(got - full).max() <= 1e-4 * np.abs(full).max()
    a = model.generate(ids[:, :5], 4, temperature=0)
    assert a.shape == (2, 9) and np.array_equal(a[:, :5], ids[:, :5])
