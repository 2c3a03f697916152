"""Launches N ranks of a module-level function as separate processes.

Each child gets RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (loopback) and
runs ``fn(rank, world, *args)``.  The parent fails with the first child's
traceback if any child exits non-zero or the timeout expires.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import socket
import traceback


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _child(fn, rank, world, port, args, extra_env, errq):
    os.environ["RANK"] = str(rank)
    os.environ["LOCAL_RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    for k, v in (extra_env or {}).items():
        os.environ[k] = v
    import faulthandler

    faulthandler.enable()
    try:
        fn(rank, world, *args)
    except BaseException:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
        raise SystemExit(1)


def run_ranks(fn, world: int, args=(), timeout: float = 180.0, extra_env=None, expect_fail=False):
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = free_port()
    procs = [
        ctx.Process(target=_child, args=(fn, r, world, port, args, extra_env, errq))
        for r in range(world)
    ]
    for p in procs:
        p.start()
    codes = []
    for p in procs:
        p.join(timeout)
        if p.is_alive():
            p.kill()
            p.join()
            codes.append("timeout")
        else:
            codes.append(p.exitcode)
    if expect_fail:
        return codes
    if any(c != 0 for c in codes):
        msgs = []
        while not errq.empty():
            r, tb = errq.get()
            msgs.append(f"--- rank {r} ---\n{tb}")
        raise AssertionError(f"ranks exited with {codes}\n" + "\n".join(msgs))
    return codes
