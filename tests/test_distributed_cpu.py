"""Host-side logic of the data-parallel path, on CPU: bucket planning, the
rendezvous that carries the NCCL id (including a rank that never arrives), the
launcher, and — with two gloo ranks — that averaging the flat gradient buffer
bucket by bucket reproduces the single-process mean of gradients."""
import multiprocessing as mp
import os
import subprocess
import sys
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plan_buckets_covers_the_buffer_exactly():
    from mytorch_b200.distributed.comm import plan_buckets
    for total, bucket in [(0, 8), (5, 8), (16, 8), (17, 8), (124_475_904, 16 * 1024 * 1024)]:
        plan = plan_buckets(total, bucket)
        assert sum(c for _, c in plan) == total
        pos = 0
        for off, cnt in plan:
            assert off == pos and 0 < cnt <= bucket
            pos += cnt


def _peer(rank, world, port, q):
    from mytorch_b200.distributed.comm import exchange_unique_id
    try:
        q.put((rank, exchange_unique_id(rank, world, "127.0.0.1", port, lambda: bytes(range(128)), timeout=20.0)))
    except Exception as e:          # noqa: BLE001
        q.put((rank, repr(e)))


def test_rendezvous_delivers_the_id_to_every_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_peer, args=(r, 3, 23457, q)) for r in (2, 1, 0)]
    for p in procs:
        p.start()
        time.sleep(0.1)           # rank 0 deliberately starts last
    got = dict(q.get(timeout=60) for _ in range(3))
    for p in procs:
        p.join(timeout=30)
    assert all(got[r] == bytes(range(128)) for r in range(3)), got


def test_rendezvous_times_out_when_a_rank_never_arrives():
    from mytorch_b200.distributed.comm import exchange_unique_id
    t0 = time.time()
    with pytest.raises(TimeoutError):
        exchange_unique_id(0, 2, "127.0.0.1", 23458, lambda: bytes(128), timeout=1.5)
    assert time.time() - t0 < 10
    with pytest.raises(TimeoutError):
        exchange_unique_id(1, 2, "127.0.0.1", 23459, lambda: bytes(128), timeout=1.5)


def test_launcher_sets_rank_env_and_propagates_failure(tmp_path):
    from mytorch_b200.distributed.launch import launch
    script = tmp_path / "w.py"
    script.write_text(
        "import os, sys\n"
        "open(sys.argv[1] + os.environ['RANK'], 'w').write(os.environ['WORLD_SIZE'] + ' ' + os.environ['LOCAL_RANK'])\n"
        "sys.exit(3 if (len(sys.argv) > 2 and os.environ['RANK'] == '1') else 0)\n")
    assert launch(2, str(script), [str(tmp_path / "out")], master_port=23460) == 0
    assert (tmp_path / "out0").read_text() == "2 0" and (tmp_path / "out1").read_text() == "2 1"
    assert launch(2, str(script), [str(tmp_path / "o"), "fail"], master_port=23461) == 3


def _gloo_rank(rank, world, port, out):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from mytorch_b200.distributed.comm import plan_buckets
    from oracle import gpt2 as og
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    cfg = og.GPT2Config(vocab_size=50, max_seq_len=16, embed_dim=32, mlp_ratio=4, num_blocks=1, num_heads=2)
    params = og.init_params(cfg, seed=2)
    rng = np.random.default_rng(9)
    batches = [og.synthetic_batch(rng, 2, 16, 50) for _ in range(world)]
    x, y = batches[rank]
    _, _, cache = og.forward(params, cfg, x, y)
    grads = og.backward(params, cfg, cache)
    flat = np.concatenate([grads[k].reshape(-1) for k in sorted(grads)]).astype(np.float32)
    t = torch.from_numpy(flat)
    for off, cnt in plan_buckets(flat.size, 1000):       # bucket-by-bucket mean, as the GPU path does
        seg = t[off:off + cnt]
        dist.all_reduce(seg, op=dist.ReduceOp.SUM)
        seg /= world
    if rank == 0:
        want = None
        for bx, by in batches:
            _, _, c = og.forward(params, cfg, bx, by)
            g = og.backward(params, cfg, c)
            f = np.concatenate([g[k].reshape(-1) for k in sorted(g)])
            want = f if want is None else want + f
        np.savez(out, got=t.numpy(), want=(want / world).astype(np.float32))
    dist.destroy_process_group()


def test_bucketed_mean_of_gradients_with_two_gloo_ranks(tmp_path):
    ctx = mp.get_context("spawn")
    out = str(tmp_path / "g.npz")
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, 23462, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    d = np.load(out)
    assert np.abs(d["got"] - d["want"]).max() <= 1e-6 * max(1.0, np.abs(d["want"]).max())
