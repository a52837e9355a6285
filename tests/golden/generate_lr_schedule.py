"""Golden learning-rate curves from the UNMODIFIED reference scheduler
(mytorch/optim/lr_scheduler.py:60-90), written to tests/golden/cosine_lr.json.

    python tests/golden/generate_lr_schedule.py --reference /path/to/MyTorch

The scheduler only calls `optimizer._update_lr(lr)`, so a recording stub stands
in for the optimizer. `_cupy_standin/` makes the reference package import on a
machine without CuPy. The tests read only the .json file.
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = [  # (max_lr, min_lr, total_steps, warmup_steps, steps to run)
    (6e-4, 6e-5, 50, 10, 60),
    (3e-4, 0.0, 20, 0, 20),
    (1e-3, 1e-4, 8, 8, 12),
]


class Recorder:
    def __init__(self):
        self.lrs = []

    def _update_lr(self, lr):
        self.lrs.append(lr)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (read only)")
    args = ap.parse_args()
    sys.path[:0] = [os.path.join(HERE, "_cupy_standin"), args.reference]
    from mytorch.optim.lr_scheduler import CosineLRScheduler
    out = []
    for max_lr, min_lr, total, warm, n in CASES:
        rec = Recorder()
        sch = CosineLRScheduler(rec, max_lr=max_lr, min_lr=min_lr, total_steps=total, warmup_steps=warm)
        for _ in range(n):
            sch.step()
        out.append({"max_lr": max_lr, "min_lr": min_lr, "total_steps": total, "warmup_steps": warm, "lrs": rec.lrs})
    with open(os.path.join(HERE, "cosine_lr.json"), "w") as fh:
        json.dump(out, fh, indent=1)
    print("wrote cosine_lr.json")


if __name__ == "__main__":
    main()
