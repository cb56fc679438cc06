"""Collective node on 2+ GPUs (child processes, one rank per GPU): the NCCL path and the
library's own P2P two-shot kernel both equal the oracle's rank-ordered sum."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _gpu_count():
    import torch
    return torch.cuda.device_count()


def _rank_main(rank, world, algo_name, count, dtype_name):
    import ctypes as C

    import torch.distributed as dist

    import habu_b200 as hb
    import oracle
    from habu_b200 import model_ir
    from mp_util import RankGuard, init_group
    init_group("gloo", rank, world)
    guard = RankGuard()
    ctx = None
    with guard:
        ctx = hb.Context(rank)
        ctx.comm_set_wait_limit(1 << 22)      # about a second: a rank that stops early costs its peers little
        # rendezvous over the host channel: NCCL id, then IPC handles
        ids = [hb.Context.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        ctx.comm_init_rank(world, rank, ids[0])
        es = 2 if dtype_name == "bf16" else 4
        nbytes = count * es
        ptr, handle = ctx.p2p_alloc(nbytes)
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        ctx.p2p_attach(world, rank, handles, nbytes)
        dtype = hb.HB_BF16 if dtype_name == "bf16" else hb.HB_F32
        algo = {"nccl": hb.HB_AR_NCCL, "p2p": hb.HB_AR_P2P, "auto": hb.HB_AR_AUTO}[algo_name]
        per_rank = [oracle.normal((count,), 900 + r) for r in range(world)]
        if dtype_name == "bf16":
            per_rank = [oracle.round_bf16(x) for x in per_rank]
        mine = per_rank[rank]
        host = oracle.to_bf16_bits(mine) if dtype_name == "bf16" else mine
        x = ctx.wrap(ptr, (count,), dtype)
        ref = per_rank[0].astype(np.float32).copy()
        for r in range(1, world):
            ref = ref + per_rank[r]
    ok = guard.agree()
    for rep in range(3 if ok else 0):            # repeated calls reuse the flag words with growing epochs
        with guard:
            ctx._check(model_ir._lib.hb_upload(ctx._h, x.ptr, host.ctypes.data_as(C.c_void_p), host.nbytes))
            ctx.sync()
        if not guard.agree():                    # every rank's input is in place (or everybody stops)
            break
        with guard:
            ctx.all_reduce(x, algo)
            ctx.sync()
            got = ctx.download(x)
            got = oracle.from_bf16_bits(got) if dtype_name == "bf16" else got
            if dtype_name == "bf16":
                # the P2P kernel adds in fp32 in rank order and rounds once; NCCL may round per hop
                tol = 2.0 ** -7 * np.maximum(np.abs(ref), 1.0)
                assert np.all(np.abs(got - ref) <= tol), float(np.abs(got - ref).max())
                if algo_name != "nccl":
                    assert np.array_equal(got, oracle.round_bf16(ref.copy()))
            else:
                assert np.allclose(got, ref, rtol=1e-6, atol=1e-6)
        if not guard.agree():
            break
        with guard:
            gathered = [None] * world
            dist.all_gather_object(gathered, got.tobytes())
            assert all(g == gathered[0] for g in gathered), "ranks disagree"
        if not guard.agree():
            break
    # the same tear-down on every rank, whatever happened above
    if ctx is not None:
        ctx.close()
    dist.barrier()
    dist.destroy_process_group()
    guard.reraise()


@pytest.mark.parametrize("algo,count,dtype", [("p2p", 1 << 20, "bf16"), ("p2p", 1000003, "bf16"), ("p2p", 77, "f32"),
                                              ("nccl", 1 << 20, "bf16"), ("auto", 8192 * 512, "bf16")])
def test_all_reduce_across_ranks(algo, count, dtype):
    n = _gpu_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    from mp_util import run_ranks
    run_ranks(_rank_main, min(n, 4) if n >= 4 else 2, (algo, count, dtype))


def test_single_rank_all_reduce_is_identity(ctx):
    import habu_b200 as hb
    import oracle
    x = oracle.to_bf16_bits(oracle.normal((1000,), 5))
    d = ctx.upload(x)
    ctx.all_reduce(d)
    assert np.array_equal(ctx.download(d), x)


def _nvls_rank(rank, world, count, dtype_name):
    """In-switch reduction over a multicast mapping.  The symmetric buffer and its multicast
    mapping come from torch's symmetric-memory allocator (plumbing only); the reduction is
    this library's multimem kernel.  No rank leaves while its memory is bound to the
    multicast object: failures are voted on over a gloo group and every rank runs the same
    tear-down."""
    import ctypes as C

    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm

    import habu_b200 as hb
    import oracle
    from habu_b200 import model_ir
    from mp_util import RankGuard, init_group
    torch.cuda.set_device(rank)
    init_group("nccl", rank, world, device_id=torch.device("cuda", rank))
    guard = RankGuard(dist.new_group(backend="gloo"))
    ctx = buf = hdl = None
    have_mc = False
    with guard:
        ctx = hb.Context(rank)
        ctx.comm_set_wait_limit(1 << 22)
        es = 2 if dtype_name == "bf16" else 4
        payload = (count * es + 255) // 256 * 256
        buf = symm.empty(payload + hb.Context.p2p_flag_bytes(), dtype=torch.uint8, device=f"cuda:{rank}")
        buf.zero_()
        hdl = symm.rendezvous(buf, dist.group.WORLD)
        torch.cuda.synchronize()
        have_mc = bool(hdl.multicast_ptr)
        if have_mc:
            ctx.p2p_attach_external(world, rank, list(hdl.buffer_ptrs), hdl.multicast_ptr, count * es)
            dtype = hb.HB_BF16 if dtype_name == "bf16" else hb.HB_F32
            per_rank = [oracle.normal((count,), 700 + r) for r in range(world)]
            if dtype_name == "bf16":
                per_rank = [oracle.round_bf16(x) for x in per_rank]
            host = oracle.to_bf16_bits(per_rank[rank]) if dtype_name == "bf16" else per_rank[rank]
            x = ctx.wrap(hdl.buffer_ptrs[rank], (count,), dtype)
            ref = per_rank[0].astype(np.float32).copy()
            for r in range(1, world):
                ref = ref + per_rank[r]
        elif rank == 0:
            print("no multicast support on this box: NVLS path not exercised")
    ok = guard.agree() and have_mc
    for algo in ((hb.HB_AR_NVLS, hb.HB_AR_P2P, hb.HB_AR_AUTO) if ok else ()):
        with guard:
            ctx._check(model_ir._lib.hb_upload(ctx._h, x.ptr, host.ctypes.data_as(C.c_void_p), host.nbytes))
            ctx.sync()
        if not guard.agree():
            break
        with guard:
            ctx.all_reduce(x, algo)
            ctx.sync()
            got = ctx.download(x)
            got = oracle.from_bf16_bits(got) if dtype_name == "bf16" else got
            tol = 2.0 ** -7 * np.maximum(np.abs(ref), 1.0) if dtype_name == "bf16" else 1e-5 * np.maximum(np.abs(ref), 1.0)
            assert np.all(np.abs(got - ref) <= tol), (algo, float(np.abs(got - ref).max()))
        if not guard.agree():
            break
        with guard:
            gathered = [None] * world
            dist.all_gather_object(gathered, got.tobytes(), group=guard.group)
            assert all(g == gathered[0] for g in gathered), "ranks disagree"
        if not guard.agree():
            break
    # tear-down in the same order on every rank: kernels drained, context closed, then a
    # barrier so that nobody releases the symmetric buffer while a peer may still use it
    if ctx is not None:
        ctx.close()
    torch.cuda.synchronize()
    dist.barrier(group=guard.group)
    del hdl, buf
    dist.barrier(group=guard.group)
    dist.destroy_process_group()
    guard.reraise()


@pytest.mark.parametrize("count,dtype", [(1 << 20, "bf16"), (100003, "bf16"), (4099, "f32")])
def test_in_switch_all_reduce_over_multicast(count, dtype):
    n = _gpu_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    from mp_util import run_ranks
    run_ranks(_nvls_rank, min(n, 4) if n >= 4 else 2, (count, dtype))
