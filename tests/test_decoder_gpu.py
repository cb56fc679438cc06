"""Decoder block forward through the model-IR executor: 1 GPU against the CPU oracle,
and 2 tensor-parallel ranks against both the oracle and each other.

Tolerances: against the oracle in bf16-storage mode (same rounding points) max-abs 2e-2
plus one bf16 output rounding; against the pure-fp32 oracle max-abs 4e-2 plus one output
rounding (two layers of bf16 residual-stream roundings sit between the two).  The small
configuration keeps the oracle's run time to seconds."""
import numpy as np
import pytest

import oracle
from habu_b200.tp import DecoderConfig, DecoderGraph, shard_layer
from oracle import decoder
from util import bf16_close

pytestmark = pytest.mark.gpu
CFG = DecoderConfig(d_model=512, n_q_heads=4, n_kv_heads=2, head_dim=128, ffn_hidden=1024, n_layers=2, batch=2, seq=256)


def _bits(layer):
    return {k: oracle.to_bf16_bits(v) for k, v in layer.items()}


def test_single_gpu_forward_matches_oracle(ctx):
    layers = [decoder.make_layer(CFG, i) for i in range(CFG.n_layers)]
    x0 = decoder.make_input(CFG)
    dg = DecoderGraph(ctx, CFG, 1, 0, [_bits(shard_layer(l, CFG, 1, 0)) for l in layers])
    arena, sym = dg.plan()
    text = dg.graph.describe()
    assert "n0 rmsnorm" in text and "all_reduce" in text and f"arena {arena}" in text
    import ctypes as C
    from habu_b200 import model_ir
    xb = oracle.to_bf16_bits(x0)
    ctx._check(model_ir._lib.hb_upload(ctx._h, dg.x0.ptr, xb.ctypes.data_as(C.c_void_p), xb.nbytes))
    for _ in range(2):                       # running twice must give the same answer (no stale state)
        dg.run()
        ctx.sync()
        got = oracle.from_bf16_bits(ctx.download(dg.out))
        ref = decoder.forward(CFG, x0, layers, round_bf16=True)
        assert bf16_close(got, ref) < 0
    ref32 = decoder.forward(CFG, x0, layers, round_bf16=False)
    assert bf16_close(got, ref32, atol=4e-2) < 0
    # the planner reuses memory: the arena is smaller than the sum of all temporaries
    total = sum(int(l.split("bytes ")[1].split()[0]) for l in text.splitlines() if l.startswith("t"))
    assert arena < total
    # micro-batched graph (2 chunks) computes the same values
    dg2 = DecoderGraph(ctx, CFG, 1, 0, [_bits(shard_layer(l, CFG, 1, 0)) for l in layers], chunks=2)
    dg2.plan()
    ctx._check(model_ir._lib.hb_upload(ctx._h, dg2.x0.ptr, xb.ctypes.data_as(C.c_void_p), xb.nbytes))
    dg2.run()
    ctx.sync()
    assert np.array_equal(oracle.from_bf16_bits(ctx.download(dg2.out)), got)


def _tp_rank(rank, world):
    import ctypes as C

    import torch.distributed as dist

    import habu_b200 as hb
    from habu_b200 import model_ir
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = hb.Context(rank)
    ids = [hb.Context.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    ctx.comm_init_rank(world, rank, ids[0])
    layers = [decoder.make_layer(CFG, i) for i in range(CFG.n_layers)]
    x0 = decoder.make_input(CFG)
    ref = decoder.forward(CFG, x0, layers, round_bf16=True)
    xb = oracle.to_bf16_bits(x0)
    outs = {}
    cases = [("nccl", hb.HB_AR_NCCL, 1), ("p2p", hb.HB_AR_AUTO, 1), ("p2p-overlap", hb.HB_AR_AUTO, 2),
             ("p2p-fused", hb.HB_AR_AUTO, 1)]
    graphs = {}
    need = 0
    for name, algo, chunks in cases:
        dg = DecoderGraph(ctx, CFG, world, rank, [_bits(shard_layer(l, CFG, world, rank)) for l in layers], algo, chunks,
                          fused=name.endswith("fused"))
        _, sym = dg.plan()
        need = max(need, sym)
        graphs[name] = dg
    for name, algo, chunks in cases:
        dg = graphs[name]
        if name == "p2p":
            ptr, handle = ctx.p2p_alloc(need)
            handles = [None] * world
            dist.all_gather_object(handles, handle)
            ctx.p2p_attach(world, rank, handles, need)
        if name != "nccl":
            dg.plan()                       # re-plan: allreduce operands now live in the peer-mapped buffer
            assert "sym+" in dg.graph.describe()
        ctx._check(model_ir._lib.hb_upload(ctx._h, dg.x0.ptr, xb.ctypes.data_as(C.c_void_p), xb.nbytes))
        ctx.sync()
        dist.barrier()
        for _ in range(2):
            dg.run()
        ctx.sync()
        got = oracle.from_bf16_bits(ctx.download(dg.out))
        assert bf16_close(got, ref) < 0, name
        outs[name] = got
        gathered = [None] * world
        dist.all_gather_object(gathered, got.tobytes())
        assert all(g == gathered[0] for g in gathered), "ranks disagree"
        dist.barrier()
    assert np.array_equal(outs["p2p"], outs["p2p-overlap"]), "chunked overlap changed the result"
    # the fused reduce-scatter / norm / all-gather nodes round at the same points
    assert np.array_equal(outs["p2p"], outs["p2p-fused"]), "fused collective changed the result"
    ctx.close()
    dist.destroy_process_group()


def test_two_tensor_parallel_ranks_match_oracle():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    from mp_util import run_ranks
    run_ranks(_tp_rank, 2)
