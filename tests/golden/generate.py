"""Generate the golden vectors under tests/golden/ by running the UNMODIFIED
reference (its NumPy CPU path) on seeded inputs.

Run where the reference checkout is available:

    python tests/golden/generate.py --reference /path/to/MyTorch [--steps 50]

The reference imports `cupy` unconditionally; `_cupy_standin/` (next to this
script) is a NumPy-backed stand-in that makes it import and select its CPU
path. Nothing here is imported by the product or by the GPU tests: the tests
read only the .npz/.json files this script writes.

Inputs are drawn from `np.random.default_rng(seed)` in a fixed order that the
tests repeat (see `op_inputs`), so only outputs and a few small inputs are
stored.
"""
import argparse
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def op_inputs(seed=1):
    """Seeded small-shape inputs shared by the generator and the tests."""
    r = np.random.default_rng(seed)
    f = lambda *s: r.standard_normal(s).astype(np.float32)
    d = {}
    d["ln_x"], d["ln_g"], d["ln_b"], d["ln_dy"] = f(37, 96), f(96), f(96), f(37, 96)
    d["rms_x"], d["rms_g"], d["rms_dy"] = f(29, 128), f(128), f(29, 128)
    d["sm_x"], d["sm_dy"] = f(33, 200), f(33, 200)
    d["lin_x"], d["lin_w"], d["lin_b"], d["lin_dy"] = f(48, 72), f(40, 72), f(40), f(48, 40)
    d["act_x"], d["act_dy"] = f(31, 50), f(31, 50)
    d["ce_x"] = f(41, 131)
    lab = r.integers(0, 131, 41).astype(np.int32)
    lab[[3, 17]] = -100
    d["ce_y"] = lab
    d["emb_w"] = f(23, 40)
    d["emb_idx"] = r.integers(0, 23, (5, 11)).astype(np.int32)
    d["emb_dy"] = f(5, 11, 40)
    d["at_q"], d["at_k"], d["at_v"], d["at_do"] = (f(2, 3, 70, 32) for _ in range(4))
    d["rope_x"], d["rope_dy"] = f(2, 19, 3, 32), f(2, 19, 3, 32)
    d["adam_p"], d["adam_g"] = f(257), f(3, 257)
    return d


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (read only)")
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--skip-train", action="store_true")
    args = ap.parse_args()

    sys.path[:0] = [os.path.join(HERE, "_cupy_standin"), args.reference,
                    os.path.join(args.reference, "gpt2_trainer"), ROOT]
    import mytorch
    import mytorch.nn as nn
    import mytorch.nn.functional as F
    import mytorch.optim as optim
    from mytorch import Tensor

    def T(a, grad=True):
        return Tensor(np.array(a, copy=True), requires_grad=grad)

    def npy(t):
        a = t.numpy() if hasattr(t, "numpy") else t
        return np.asarray(a)

    def g(t):
        return npy(t.grad)

    d = op_inputs()
    out = {}

    # LayerNorm (manual path), with and without bias
    x, w, b = T(d["ln_x"]), T(d["ln_g"]), T(d["ln_b"])
    y = F.layernorm(x, w, b, eps=1e-5)
    y.backward(d["ln_dy"])
    out.update(ln_y=npy(y), ln_dx=g(x), ln_dg=g(w), ln_db=g(b))
    x, w = T(d["ln_x"]), T(d["ln_g"])
    y = F.layernorm(x, w, None, eps=1e-5)
    y.backward(d["ln_dy"])
    out.update(ln_nb_y=npy(y), ln_nb_dx=g(x), ln_nb_dg=g(w))

    # RMSNorm, with weight and parameter-free
    x, w = T(d["rms_x"]), T(d["rms_g"])
    y = F.rmsnorm(x, w, eps=1e-5)
    y.backward(d["rms_dy"])
    out.update(rms_y=npy(y), rms_dx=g(x), rms_dg=g(w))
    x = T(d["rms_x"])
    y = F.rmsnorm(x, None, eps=1e-5)
    y.backward(d["rms_dy"])
    out.update(rms_nw_y=npy(y), rms_nw_dx=g(x))

    # Softmax
    x = T(d["sm_x"])
    y = F.softmax(x, dim=-1)
    y.backward(d["sm_dy"])
    out.update(sm_y=npy(y), sm_dx=g(x))

    # Linear with bias
    x, w, b = T(d["lin_x"]), T(d["lin_w"]), T(d["lin_b"])
    y = F.linear(x, w, b)
    y.backward(d["lin_dy"])
    out.update(lin_y=npy(y), lin_dx=g(x), lin_dw=g(w), lin_db=g(b))

    # GELU (manual) and ReLU^2 (auto path: the manual one has a zero gradient)
    x = T(d["act_x"])
    y = F.gelu(x)
    y.backward(d["act_dy"])
    out.update(gelu_y=npy(y), gelu_dx=g(x))
    x = T(d["act_x"])
    y = F.relu_squared(x, auto=True)
    y.backward(d["act_dy"])
    out.update(relu2_y=npy(y), relu2_dx=g(x))

    # Cross entropy with two ignored rows
    x = T(d["ce_x"])
    y = F.cross_entropy(x, T(d["ce_y"], grad=False))
    y.backward()
    out.update(ce_loss=npy(y), ce_dx=g(x))

    # Embedding (auto path: indexing + np.add.at)
    w = T(d["emb_w"])
    y = F.embedding(d["emb_idx"], w) if False else w[d["emb_idx"]]
    y.backward(d["emb_dy"])
    out.update(emb_y=npy(y), emb_dw=g(w))

    # Causal attention, composed as in the un-fused branch of gpt2.py:187-203
    q, k, v = T(d["at_q"]), T(d["at_k"]), T(d["at_v"])
    S = q.shape[-2]
    mask = np.triu(np.full((S, S), -np.inf, dtype=np.float32), k=1)[None, None]
    scores = (q @ k.transpose(-2, -1)) / (q.shape[-1] ** 0.5)
    scores = scores + Tensor(mask)
    p = F.softmax(scores, dim=-1)
    o = p @ v
    o.backward(d["at_do"])
    out.update(at_o=npy(o), at_dq=g(q), at_dk=g(k), at_dv=g(v))

    # RoPE (auto path)
    from mytorch.nn.functional.other.rotary_embeddings import (
        precompute_rotary_cos_sin, auto_apply_rotary_pos_embed)
    cos, sin = precompute_rotary_cos_sin(32, max_position_embeddings=19)
    x = T(d["rope_x"])
    x2 = T(d["rope_x"])
    qe, ke = auto_apply_rotary_pos_embed(x, x2, cos, sin)
    qe.backward(d["rope_dy"])
    out.update(rope_y=npy(qe), rope_dx=g(x), rope_cos=npy(cos)[0], rope_sin=npy(sin)[0])

    # AdamW, three steps, weight decay 0.1 (group form as in train_gpt2.py:271-285)
    p = T(d["adam_p"])
    opt = optim.AdamW([{"params": [p], "weight_decay": 0.1}], lr=3e-3, beta1=0.9, beta2=0.95)
    traj = []
    for i in range(3):
        p.grad = mytorch.Tensor(d["adam_g"][i]).data
        opt.step()
        traj.append(npy(p).copy())
    out.update(adam_p=np.stack(traj),
               adam_m=np.asarray(npy(opt.param_groups[0]["m"][0])),
               adam_v=np.asarray(npy(opt.param_groups[0]["v"][0])))

    np.savez_compressed(os.path.join(HERE, "ops_small.npz"),
                        **{k: np.asarray(v, dtype=np.float32) for k, v in out.items()})
    print("wrote ops_small.npz with", len(out), "arrays")

    if args.skip_train:
        return

    # ---- tiny GPT-2, fp32, 50 AdamW steps: loss trajectory + weight checks ----
    from gpt2 import GPT2, GPT2Config
    from oracle import gpt2 as og
    ocfg = og.GPT2Config(vocab_size=65, max_seq_len=256, embed_dim=256, mlp_ratio=4,
                         num_blocks=4, num_heads=4)
    params = og.init_params(ocfg, seed=0)
    model = GPT2(GPT2Config(vocab_size=65, max_seq_len=256, embed_dim=256, mlp_ratio=4,
                            num_blocks=4, num_heads=4, use_bias=False))
    sd = dict(params)
    sd["lm_head.weight"] = params["embeddings.char_embeddings.weight"]
    model.load_state_dict(sd)
    model.lm_head.weight = model.embeddings.char_embeddings.weight  # keep the tie
    decay, no_decay = [], []
    for name, prm in model.named_parameters():
        (no_decay if len(prm.shape) < 2 else decay).append(prm)
    opt = optim.AdamW([{"params": decay, "weight_decay": 0.1},
                       {"params": no_decay, "weight_decay": 0.0}],
                      lr=3e-4, beta1=0.9, beta2=0.95)
    loss_fn = nn.CrossEntropyLoss()
    rng = np.random.default_rng(0)
    losses, times = [], []
    first_grads = None
    for step in range(args.steps):
        xb, yb = og.synthetic_batch(rng, 16, 256, 65)
        t0 = time.perf_counter()
        logits = model(mytorch.Tensor(xb))
        loss = loss_fn(logits, mytorch.Tensor(yb))
        loss.backward()
        if step == 0:
            first_grads = {n: np.asarray(npy(p_.grad), dtype=np.float32).copy()
                           for n, p_ in model.named_parameters()}
        opt.step()
        opt.zero_grad()
        times.append(time.perf_counter() - t0)
        losses.append(float(npy(loss)))
        print(f"step {step} loss {losses[-1]:.6f} {times[-1]:.2f}s", flush=True)
    final = model.state_dict()
    summary = {
        "config": "tiny GPT-2 fp32: L4 H4 d256 ctx256 vocab65 batch16, AdamW lr3e-4 b(0.9,0.95) wd0.1",
        "losses": losses,
        "sec_per_step_here": float(np.median(times[1:])) if len(times) > 1 else times[0],
        "final_weight_l2": {k: float(np.sqrt(np.sum(np.asarray(v, dtype=np.float64) ** 2)))
                            for k, v in final.items()},
        "first_step_grad_l2": {k: float(np.sqrt(np.sum(v.astype(np.float64) ** 2)))
                               for k, v in first_grads.items()},
    }
    with open(os.path.join(HERE, "tiny_gpt2_fp32.json"), "w") as fh:
        json.dump(summary, fh, indent=1)
    # a few whole first-step gradients, small enough to commit
    keep = ["blocks.0.layernorm1.weight", "final_layer_norm.bias", "final_layer_norm.weight",
            "embeddings.char_embeddings.weight", "blocks.3.attention.out_proj.weight"]
    np.savez_compressed(os.path.join(HERE, "tiny_gpt2_first_grads.npz"),
                        **{k: first_grads[k] for k in keep})
    print("wrote tiny_gpt2_fp32.json")


if __name__ == "__main__":
    main()
