"""Worker for tests/test_ddp_gpu.py: one rank of a data-parallel run of a tiny
GPT-2 (fp32 so the comparison is tight). Rank r consumes batches r, r+W, ...;
rank 0 writes losses and final master weights to the path in argv[1]."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def run(out_path, world, rank, steps=3, accum=1, mixed=False):
    import mytorch_b200 as mt
    from mytorch_b200.gpt2 import GPT2, GPT2Config
    from oracle import gpt2 as og
    cfg = og.GPT2Config(vocab_size=96, max_seq_len=32, embed_dim=64, mlp_ratio=4, num_blocks=2, num_heads=2)
    params = og.init_params(cfg, seed=11)
    acc = mt.Accelerator(num_gpus=world, rank=rank, gradient_accumulation_steps=accum, mixed_precision=mixed)
    np.random.seed(0)
    model = GPT2(GPT2Config(vocab_size=96, max_seq_len=32, embed_dim=64, num_blocks=2, num_heads=2))
    sd = {k: v.copy() for k, v in params.items()}
    sd["lm_head.weight"] = sd["embeddings.char_embeddings.weight"]
    if rank != 0:      # only rank 0 holds the real weights: prepare() must broadcast them
        sd = {k: np.zeros_like(v) for k, v in sd.items()}
    model.load_state_dict(sd)
    decay = [p for _, p in model.named_parameters() if len(p.shape) >= 2]
    rest = [p for _, p in model.named_parameters() if len(p.shape) < 2]
    opt = mt.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0}], lr=1e-3)
    model, opt = acc.prepare(model, opt)
    loss_fn = mt.nn.CrossEntropyLoss()
    rng = np.random.default_rng(3)
    batches = [og.synthetic_batch(rng, 2, 32, 96) for _ in range(steps * 2)]   # two micro-batches per optimizer step
    losses = []
    per_step = len(batches) // steps
    for s in range(steps):
        group = batches[s * per_step:(s + 1) * per_step]
        mine = group[rank::world] if world > 1 else group
        for x, y in mine:
            loss = loss_fn(model(mt.Tensor(x)), mt.Tensor(y))
            acc.backward(loss)
            acc.clip_grad_norm_(1.0)
            opt.step()
            opt.zero_grad()
            losses.append(acc.gather_for_metrics(loss).item())
    if rank == 0:
        np.savez(out_path, losses=np.array(losses), master=acc._flat.master.numpy(), norm=acc.grad_norm)
    acc.end_training()


if __name__ == "__main__":
    out = sys.argv[1]
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    accum = int(sys.argv[2]) if len(sys.argv) > 2 else 1
    run(out, world, rank, accum=accum)
