"""Spawn helper for multi-process tests: N child processes on one host, a parent
watchdog with a timeout, identical exit codes required (the pattern of the
reference's TestDistBackend, test/cnnl/test_distributed.py:657-775)."""
import os
import socket
import sys
import traceback

import torch.multiprocessing as mp


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, fn_module, fn_name, args, env):
    os.environ.update(env)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["LOCAL_RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        mod = __import__(fn_module)
        getattr(mod, fn_name)(rank, world, *args)
    except SystemExit:
        raise
    except BaseException:
        traceback.print_exc()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(17)


def run_ranks(fn, world=2, args=(), timeout=120, env=None, expect_exit=0):
    """Run ``fn(rank, world, *args)`` in ``world`` processes; fail on timeout or wrong exit code."""
    ctx = mp.get_context("spawn")
    port = free_port()
    procs = []
    for r in range(world):
        p = ctx.Process(target=_entry, args=(r, world, port, fn.__module__, fn.__name__, args, env or {}))
        p.start()
        procs.append(p)
    codes = []
    for p in procs:
        p.join(timeout)
        if p.is_alive():
            for q in procs:
                if q.is_alive():
                    q.kill()  # exact child handles, not a pattern
            raise AssertionError(f"rank process timed out after {timeout}s")
        codes.append(p.exitcode)
    if expect_exit is not None:
        assert all(c == expect_exit for c in codes), f"exit codes {codes}"
    return codes
