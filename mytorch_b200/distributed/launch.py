"""One process per GPU on a single node, like
`python -m mytorch.distributed.launch --num_gpus N script.py args...`
(mytorch/distributed/launch.py:7-58): each child gets RANK, LOCAL_RANK,
WORLD_SIZE, CUPYX_DISTRIBUTED_HOST/PORT; Ctrl-C or a failing child stops the
others (each child runs in its own process group)."""
import argparse
import os
import signal
import subprocess
import sys
import time


def launch(num_gpus, script, script_args, master_addr="127.0.0.1", master_port=13333, extra_env=None, poll=0.2):
    procs = []
    for rank in range(num_gpus):
        env = dict(os.environ)
        env.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(num_gpus),
                    "CUPYX_DISTRIBUTED_HOST": master_addr, "CUPYX_DISTRIBUTED_PORT": str(master_port)})
        if extra_env:
            env.update(extra_env)
        procs.append(subprocess.Popen([sys.executable, script, *script_args], env=env, start_new_session=True))

    def stop_all():
        for p in procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)   # exactly the group we started
                except ProcessLookupError:
                    pass

    rc = 0
    try:
        alive = set(range(num_gpus))
        while alive:
            for r in list(alive):
                code = procs[r].poll()
                if code is not None:
                    alive.discard(r)
                    if code != 0:
                        rc = rc or code
                        stop_all()
            time.sleep(poll)
    except KeyboardInterrupt:
        stop_all()
        rc = 130
    return rc


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--num_gpus", type=int, default=1)
    ap.add_argument("--master_addr", default="127.0.0.1")
    ap.add_argument("--master_port", type=int, default=13333)
    ap.add_argument("script")
    ap.add_argument("script_args", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    return launch(a.num_gpus, a.script, a.script_args, a.master_addr, a.master_port)


if __name__ == "__main__":
    sys.exit(main())
