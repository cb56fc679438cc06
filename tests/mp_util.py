"""Runs a function as `world` ranks in child processes (one per GPU, or CPU ranks over
gloo) and re-raises the first failure.

A rank that fails must not simply exit: its peers would stay blocked in their next
collective until they are killed, and a killed rank may still hold peer-mapped or
multicast-bound memory.  `RankGuard` is the protocol the rank bodies follow instead: work is
done in guarded steps, a failure inside a step is recorded rather than raised, and after
every step the ranks agree over the host channel (a gloo group) whether anyone failed.  If
so, every rank stops issuing collectives, runs the same tear-down (close the context, free
the symmetric buffer, destroy the process group) and only then re-raises."""
import datetime
import multiprocessing as mp
import os
import tempfile
import traceback


def init_group(backend, rank, world, **kw):
    """init_process_group over a file store.  A TCP store needs a port that is picked before the
    ranks start and can be taken by somebody else before rank 0 binds it (seen once: rank 0 died
    with EADDRINUSE and its peer sat in the rendezvous until the harness gave up); a file needs
    none.  The short timeout makes a rank whose peer never arrives fail within two minutes."""
    import torch.distributed as dist
    dist.init_process_group(backend, init_method="file://" + os.environ["HB_TEST_RDZV_FILE"], rank=rank,
                            world_size=world, timeout=datetime.timedelta(seconds=120), **kw)


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


def _entry(fn, rank, world, rdzv, q, args):
    os.environ.update({"HB_TEST_RDZV_FILE": rdzv, "RANK": str(rank), "WORLD_SIZE": str(world),
                       "LOCAL_RANK": str(rank)})
    try:
        fn(rank, world, *args)
        q.put((rank, None))
    except BaseException:
        q.put((rank, traceback.format_exc()))


def run_ranks(fn, world, args=(), timeout=300):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    rdzv_dir = tempfile.mkdtemp(prefix="hb_rdzv_")
    rdzv = os.path.join(rdzv_dir, "store")
    procs = [ctx.Process(target=_entry, args=(fn, r, world, rdzv, q, args)) for r in range(world)]
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
                timeout = min(timeout, 150)   # its peers follow within the group's own timeout, or never
            elif err:
                errors.append(f"rank {rank} stopped because a peer failed")
    finally:
        # ranks tear down by themselves; give them time, and end a process only as a last resort
        for p in procs:
            p.join(timeout=30 if errors else 120)
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=30)
                if p.is_alive():
                    p.kill()
    try:
        if os.path.exists(rdzv):
            os.unlink(rdzv)
        os.rmdir(rdzv_dir)
    except OSError:
        pass
    assert not errors, "\n".join(errors)
