"""Runs a function as `world` ranks in child processes (one per GPU, or CPU ranks over
gloo) and re-raises the first failure."""
import multiprocessing as mp
import os
import socket
import traceback


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(fn, rank, world, port, q, args):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank),
                       "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank)})
    try:
        fn(rank, world, *args)
        q.put((rank, None))
    except Exception:
        q.put((rank, traceback.format_exc()))


def run_ranks(fn, world, args=(), timeout=300):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, q, args)) for r in range(world)]
    for p in procs:
        p.start()
    errors = []
    try:
        for _ in range(world):
            rank, err = q.get(timeout=timeout)
            if err:
                errors.append(f"rank {rank}:\n{err}")
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    assert not errors, "\n".join(errors)
