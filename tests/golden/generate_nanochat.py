"""Golden vectors for the nanochat-style GPT: runs the UNMODIFIED reference
model (nanochat_trainer/core/nanochat_gpt.py, NumPy CPU path, non-fused) on two
tiny configurations with seeded weights - multi-head, and grouped-query with 4 query and
2 key/value heads - and writes tests/golden/nanochat_tiny.json and nanochat_tiny_gqa.json.

    python tests/golden/generate_nanochat.py --reference /path/to/MyTorch

The reference's CPU cross entropy cannot take a softcap, so the capped logits
come from the model's own inference branch (forward(ids, None) returns
softcap * tanh(logits / softcap)) and its plain cross entropy is applied to them.
ReLU^2 uses the reference's `auto` path (module flag), because its default path is defective.
"""
import argparse
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (read only)")
    args = ap.parse_args()
    sys.path[:0] = [os.path.join(HERE, "_cupy_standin"), args.reference,
                    os.path.join(args.reference, "nanochat_trainer", "core"), ROOT]
    import mytorch
    import mytorch.nn.functional as F
    import mytorch.optim as optim
    import mytorch.nn.functional._compat as compat
    compat.FUSED_AVAIL = False      # the reference's own switch: take its NumPy path although Triton is importable
    from nanochat_gpt import GPT, GPTConfig
    from oracle import nanochat as on
    from oracle import gpt2 as og

    cases = [("nanochat_tiny.json", dict(num_heads=2, num_kv_heads=0), 4,
              "nanochat tiny fp32: L2 H2 d64 ctx32 vocab96 batch3, AdamW lr1e-3 b(0.9,0.95) wd0.1 on all tensors"),
             ("nanochat_tiny_gqa.json", dict(num_heads=4, num_kv_heads=2), 5,
              "nanochat tiny fp32, grouped-query: L2 Hq4 Hkv2 d64 ctx32 vocab96 batch3, AdamW lr1e-3 b(0.9,0.95) wd0.1")]
    for fname, heads, seed, label in cases:
        ocfg = on.GPTConfig(vocab_size=96, max_seq_len=32, embed_dim=64, mlp_ratio=4, num_blocks=2, **heads)
        params = on.init_params(ocfg, seed=seed)
        model = GPT(GPTConfig(vocab_size=96, max_seq_len=32, embed_dim=64, mlp_ratio=4, num_blocks=2,
                              num_q_heads=heads["num_heads"], num_kv_heads=heads["num_kv_heads"] or heads["num_heads"],
                              use_fused_ops=False))
        model.load_state_dict(params)
        # ReLU^2: select the reference's `auto` implementation through the module's own switch; its
        # default `manual` one zeroes its input in place and returns a zero gradient
        # (mytorch/nn/functional/activations/relu_squared.py:13-27).
        for blk in model.blocks:
            blk.feedforward.activation.auto = True
        plist = [p for _, p in model.named_parameters()]
        opt = optim.AdamW([{"params": plist, "weight_decay": 0.1}], lr=1e-3, beta1=0.9, beta2=0.95)
        rng = np.random.default_rng(8)
        losses, first = [], None
        for step in range(6):
            x, y = og.synthetic_batch(rng, 3, 32, 96)
            capped = model(mytorch.Tensor(x), None)[0]
            loss = F.cross_entropy(capped, mytorch.Tensor(y))
            loss.backward()
            if step == 0:
                first = {n: float(np.sqrt(np.sum(np.asarray(p.grad.numpy() if hasattr(p.grad, "numpy") else p.grad, dtype=np.float64) ** 2)))
                         for n, p in model.named_parameters()}
            opt.step()
            opt.zero_grad()
            losses.append(float(np.asarray(loss.numpy())))
            print(fname, step, losses[-1], flush=True)
        final = model.state_dict()
        out = {"config": label, "losses": losses, "first_step_grad_l2": first,
               "final_weight_l2": {k: float(np.sqrt(np.sum(np.asarray(v, dtype=np.float64) ** 2))) for k, v in final.items()}}
        with open(os.path.join(HERE, fname), "w") as fh:
            json.dump(out, fh, indent=1)
        print("wrote", fname)


if __name__ == "__main__":
    main()
