"""Runs a function as `world` ranks in child processes (one per GPU, or CPU ranks over
gloo) and re-raises the first failure.

A rank that fails must not simply exit: its peers would stay blocked in their next
collective until they are killed, and a killed rank may still hold peer-mapped or
multicast-bound memory.  `RankGuard` is the protocol the rank bodies follow instead: work is
done in guarded steps, a failure inside a step is recorded rather than raised, and after
every step the ranks agree over the host channel (a gloo group) whether anyone failed.  If
so, every rank stops issuing collectives, runs the same tear-down (close the context, free
the symmetric buffer, destroy the process group) and only then re-raises."""
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


class RankGuard:
    """with guard: ...   records an exception instead of raising it;
    guard.agree()        host-side vote (gloo): True when no rank has failed so far;
    guard.reraise()      raises the recorded failure (call after the tear-down)."""

    def __init__(self, group=None):
        self.group = group
        self.error = None
        self.peer_failed = False

    def __enter__(self):
        return self

    def __exit__(self, et, ev, tb):
        if et is not None and self.error is None:
            self.error = "".join(traceback.format_exception(et, ev, tb))
        return True          # swallowed here, re-raised after the tear-down

    def agree(self) -> bool:
        import torch
        import torch.distributed as dist
        flag = torch.tensor([1 if self.error else 0], dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        if int(flag.item()) and not self.error:
            self.peer_failed = True
        return int(flag.item()) == 0

    def reraise(self):
        if self.error:
            raise AssertionError(self.error)
        if self.peer_failed:
            raise AssertionError("another rank failed; this rank stopped with it")


def _entry(fn, rank, world, port, q, args):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank),
                       "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank)})
    try:
        fn(rank, world, *args)
        q.put((rank, None))
    except BaseException:
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
            try:
                rank, err = q.get(timeout=timeout)
            except Exception:
                errors.append(f"no answer from some rank within {timeout} s")
                break
            if err and "another rank failed" not in err:
                errors.append(f"rank {rank}:\n{err}")
            elif err:
                errors.append(f"rank {rank} stopped because a peer failed")
    finally:
        # ranks tear down by themselves; give them time, and end a process only as a last resort
        for p in procs:
            p.join(timeout=120)
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=30)
                if p.is_alive():
                    p.kill()
    assert not errors, "\n".join(errors)
