"""Data-parallel parity on 2 GPUs: two ranks, each with its own micro-batch per
step, must end with the same weights as ONE process that accumulates the same
two micro-batches (mean of gradients) — the definition of parity for W > 1,
since the reference's own gradient all-reduce discards its result
(mytorch/accelerate.py:757-772). Also checks that rank 0's weights reach rank 1
(rank 1 starts from zeros). Runs as child processes started by the launcher."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "ddp_worker.py")


def test_two_ranks_match_single_process_accumulation(tmp_path):
    from mytorch_b200 import _lib
    if _lib.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from mytorch_b200.distributed.launch import launch
    ddp_out = str(tmp_path / "ddp.npz")
    single_out = str(tmp_path / "single.npz")
    rc = launch(2, WORKER, [ddp_out, "1"], master_port=13571, extra_env={"NCCL_NVLS_ENABLE": "0"})
    assert rc == 0
    env = dict(os.environ, WORLD_SIZE="1", RANK="0", LOCAL_RANK="0")
    subprocess.run([sys.executable, WORKER, single_out, "2"], env=env, check=True, timeout=300)
    a, b = np.load(ddp_out), np.load(single_out)
    assert np.abs(a["master"] - b["master"]).max() <= 1e-5 * max(1.0, np.abs(b["master"]).max())
    assert abs(float(a["norm"]) - float(b["norm"])) <= 1e-4 * float(b["norm"])
    # rank-averaged loss of step s equals the mean of the single process's two micro-batch losses
    single = b["losses"].reshape(-1, 2).mean(axis=1)
    assert np.abs(a["losses"] - single).max() <= 1e-5 * single.max()
