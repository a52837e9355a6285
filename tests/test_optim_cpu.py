"""Host-side optimiser logic that needs no GPU: the cosine learning-rate schedule against the
curves of the unmodified reference scheduler (tests/golden/cosine_lr.json, written by
tests/golden/generate_lr_schedule.py from mytorch/optim/lr_scheduler.py:60-90)."""
import json
import os

import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


class _Groups:
    """What the scheduler touches of an optimizer: a list of groups with an "lr"."""

    def __init__(self, n=2, lr=123.0):
        self.param_groups = [{"lr": lr} for _ in range(n)]


def test_cosine_schedule_matches_reference_curves():
    from mytorch_b200.optim import CosineLRScheduler
    with open(os.path.join(GOLDEN, "cosine_lr.json")) as fh:
        cases = json.load(fh)
    assert len(cases) >= 3
    for c in cases:
        opt = _Groups()
        sch = CosineLRScheduler(opt, max_lr=c["max_lr"], min_lr=c["min_lr"], total_steps=c["total_steps"],
                                warmup_steps=c["warmup_steps"])
        assert all(g["lr"] == 123.0 for g in opt.param_groups)     # untouched until the first step()
        for k, want in enumerate(c["lrs"]):
            got = sch.step()
            assert got == pytest.approx(want, rel=1e-12, abs=1e-18), (c, k)
            assert all(g["lr"] == got for g in opt.param_groups)
        # warm-up is linear up to max_lr, the end of the horizon sits at min_lr
        if c["warmup_steps"]:
            assert c["lrs"][c["warmup_steps"] - 1] == pytest.approx(c["max_lr"])
        if len(c["lrs"]) >= c["total_steps"] > c["warmup_steps"]:
            assert c["lrs"][c["total_steps"] - 1] == pytest.approx(c["min_lr"], abs=1e-12)
