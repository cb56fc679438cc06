"""Decoder block forward through the model-IR executor: 1 GPU against the CPU oracle,
and 2 tensor-parallel ranks against both the oracle and each other.

Tolerances.  Against the oracle in bf16-storage mode (it rounds the same tensors at the same
points): max-abs 2e-2 plus one bf16 output rounding -- the implementation check.  Against the
pure-fp32 oracle the flat 2e-2 that holds for a single GEMM or attention call cannot hold for
this block: its outputs reach |x| ~ 5 (small configuration) and ~ 20 (full size), where one
bf16 rounding of the OUTPUT alone is 0.016 / 0.06, and the bf16-storage oracle itself deviates
from fp32 by 0.044 / 0.18 (every rounding point contributes; keeping the residual stream in
fp32 would only bring 0.18 to 0.14).  The fp32 comparison is therefore made in units of the
output's scale: max-abs / max|ref| <= 2e-2, with the raw figures printed.  The small
configuration keeps the oracle's run time to seconds; one full-size sequence is checked too."""
import numpy as np
import pytest

import oracle
from habu_b200.tp import DecoderConfig, DecoderGraph, shard_layer
from oracle import decoder
from util import bf16_close

pytestmark = pytest.mark.gpu
CFG = DecoderConfig(d_model=512, n_q_heads=4, n_kv_heads=2, head_dim=128, ffn_hidden=1024, n_layers=2, batch=2, seq=256)


def scaled_err(got, ref32):
    """max-abs error against the fp32 oracle in units of the output's scale."""
    return float(np.max(np.abs(got - ref32)) / np.max(np.abs(ref32)))


def rel_rms(got, ref):
    d = (got - ref).astype(np.float64)
    return float(np.sqrt(np.mean(d * d)) / np.sqrt(np.mean(ref.astype(np.float64) ** 2)))


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
    assert scaled_err(got, ref32) < 2e-2
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


def _upload(ctx, dg, xb):
    import ctypes as C
    from habu_b200 import model_ir
    ctx._check(model_ir._lib.hb_upload(ctx._h, dg.x0.ptr, xb.ctypes.data_as(C.c_void_p), xb.nbytes))
    ctx.sync()


def _tp_rank(rank, world, nvls):
    """All collective variants of the tensor-parallel block on `world` GPUs.  nvls=False:
    NCCL, the library's P2P kernel, micro-batched overlap and the fused reduce-scatter/norm/
    all-gather node over a cudaIpc mapping.  nvls=True: the in-switch (multimem) allreduce and
    the in-switch fused node over a multicast mapping from torch's symmetric-memory
    allocator (plumbing only) -- the default of the benchmark's decoder workload."""
    import torch
    import torch.distributed as dist

    import habu_b200 as hb
    from mp_util import RankGuard, init_group
    torch.cuda.set_device(rank)
    init_group("nccl", rank, world, device_id=torch.device("cuda", rank))
    guard = RankGuard(dist.new_group(backend="gloo"))
    ctx = buf = hdl = None
    outs, graphs = {}, {}
    if nvls:
        cases = [("nvls", hb.HB_AR_NVLS, 1), ("nvls-fused", hb.HB_AR_NVLS, 1), ("nvls-fused-pipelined", hb.HB_AR_NVLS, 2),
                 ("nvls-fused-gathered", hb.HB_AR_NVLS, 1), ("p2p-fused", hb.HB_AR_P2P, 1)]
    else:
        cases = [("nccl", hb.HB_AR_NCCL, 1), ("p2p", hb.HB_AR_AUTO, 1), ("p2p-overlap", hb.HB_AR_AUTO, 2),
                 ("p2p-fused", hb.HB_AR_AUTO, 1), ("p2p-fused-pipelined", hb.HB_AR_AUTO, 2),
                 ("p2p-fused-gathered", hb.HB_AR_AUTO, 1)]
    have = True
    with guard:
        ctx = hb.Context(rank)
        ctx.comm_set_wait_limit(1 << 22)
        ids = [hb.Context.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0, group=guard.group)
        ctx.comm_init_rank(world, rank, ids[0])
        layers = [decoder.make_layer(CFG, i) for i in range(CFG.n_layers)]
        x0 = decoder.make_input(CFG)
        ref = decoder.forward(CFG, x0, layers, round_bf16=True)
        xb = oracle.to_bf16_bits(x0)
        need = 0
        for name, algo, chunks in cases:
            dg = DecoderGraph(ctx, CFG, world, rank, [_bits(shard_layer(l, CFG, world, rank)) for l in layers], algo, chunks,
                              fused="fused" in name, gathered="gathered" in name)
            _, sym = dg.plan()
            need = max(need, sym)
            graphs[name] = dg
        if nvls:
            import torch.distributed._symmetric_memory as symm
            payload = (need + 255) // 256 * 256
            buf = symm.empty(payload + hb.Context.p2p_flag_bytes(), dtype=torch.uint8, device=f"cuda:{rank}")
            buf.zero_()
            hdl = symm.rendezvous(buf, dist.group.WORLD)
            torch.cuda.synchronize()
            have = bool(hdl.multicast_ptr)
            if have:
                ctx.p2p_attach_external(world, rank, list(hdl.buffer_ptrs), hdl.multicast_ptr, need)
            elif rank == 0:
                print("no multicast support on this box: in-switch decoder path not exercised")
        else:
            ptr, handle = ctx.p2p_alloc(need)
            handles = [None] * world
            dist.all_gather_object(handles, handle, group=guard.group)
            ctx.p2p_attach(world, rank, handles, need)
    ok = guard.agree() and have
    for name, algo, chunks in (cases if ok else ()):
        dg = graphs[name]
        with guard:
            if name != "nccl":
                dg.plan()                       # re-plan: allreduce operands now live in the peer-mapped buffer
                assert "sym+" in dg.graph.describe()
            _upload(ctx, dg, xb)
        if not guard.agree():
            break
        with guard:
            for _ in range(2):
                dg.run()
            ctx.sync()
            got = oracle.from_bf16_bits(ctx.download(dg.out))
            # The ranks round their partial products before the sum, the oracle rounds the whole
            # product once: an output that lands on the other side of a rounding boundary moves
            # by a full bf16 ulp (2^-7 relative: 0.0625 for |x| in [8, 16), more than
            # 2e-2 + 2^-8 |x| there), so the widening is one ulp here, not the half ulp of a
            # single rounding.
            assert bf16_close(got, ref, rel=2.0 ** -7) < 0, (name, bf16_close(got, ref, rel=2.0 ** -7))
            outs[name] = got
        if not guard.agree():
            break
        with guard:
            gathered = [None] * world
            dist.all_gather_object(gathered, got.tobytes(), group=guard.group)
            assert all(g == gathered[0] for g in gathered), f"{name}: ranks disagree"
        if not guard.agree():
            break
    with guard:
        if ok and nvls and len(outs) == len(cases):
            assert np.array_equal(outs["nvls-fused"], outs["nvls-fused-gathered"]), "the gathered products changed the result"
        if ok and not nvls and len(outs) == len(cases):
            assert np.array_equal(outs["p2p"], outs["p2p-overlap"]), "chunked overlap changed the result"
            # the fused reduce-scatter / norm / all-gather nodes round at the same points
            assert np.array_equal(outs["p2p"], outs["p2p-fused"]), "fused collective changed the result"
            # row blocks pipelined over two streams: same arithmetic per row, same bits
            assert np.array_equal(outs["p2p"], outs["p2p-fused-pipelined"]), "pipelined row blocks changed the result"
            # products that wait for their gathered rows word by word: same arithmetic again
            assert np.array_equal(outs["p2p"], outs["p2p-fused-gathered"]), "the gathered products changed the result"
    # same tear-down on every rank: drain, close, and only then let the mappings go
    if ctx is not None:
        for dg in graphs.values():
            dg.graph.close()
        ctx.close()
    torch.cuda.synchronize()
    dist.barrier(group=guard.group)
    del hdl, buf
    dist.barrier(group=guard.group)
    dist.destroy_process_group()
    guard.reraise()


@pytest.mark.parametrize("nvls", [False, True], ids=["ipc", "multicast"])
def test_two_tensor_parallel_ranks_match_oracle(nvls):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    from mp_util import run_ranks
    run_ranks(_tp_rank, 2, (nvls,))


@pytest.mark.timeout(900)
def test_full_size_sequence_matches_oracle():
    """The benchmark's block at its real width (d_model 4096, 32/8 heads, FFN 14336, 2 layers):
    one sequence of 2048 tokens against the oracle in both modes."""
    import habu_b200 as hb
    from dataclasses import replace
    oracle.use_all_cores()
    cfg = replace(DecoderConfig(), batch=1)
    layers = [decoder.make_layer(cfg, i) for i in range(cfg.n_layers)]
    x0 = decoder.make_input(cfg)
    ctx = hb.Context(0)
    try:
        dg = DecoderGraph(ctx, cfg, 1, 0, [_bits(shard_layer(l, cfg, 1, 0)) for l in layers])
        dg.plan()
        _upload(ctx, dg, oracle.to_bf16_bits(x0))
        dg.run()
        ctx.sync()
        got = oracle.from_bf16_bits(ctx.download(dg.out))
    finally:
        ctx.close()
    ref = decoder.forward(cfg, x0, layers, round_bf16=True)
    ref32 = decoder.forward(cfg, x0, layers, round_bf16=False)
    print(f"full-size decoder: max-abs vs bf16-storage oracle {np.abs(got - ref).max():.4f}, vs fp32 oracle "
          f"{np.abs(got - ref32).max():.4f} (bf16-storage oracle vs fp32: {np.abs(ref - ref32).max():.4f}), "
          f"max |ref| {np.abs(ref32).max():.2f}")
    # At this depth and width (K up to 14336, |x| up to 20) two bf16 implementations with the same
    # rounding points but different summation orders differ from each other as much as either
    # differs from fp32: a rounding that flips moves a value by one bf16 ulp (0.125 near 16) and
    # the difference propagates.  So all three comparisons are made in units of the output's
    # scale, on the maximum and on the RMS (the bf16-storage oracle is at 0.0088 / 0.0075 of fp32).
    assert scaled_err(got, ref) < 2e-2 and rel_rms(got, ref) < 1.5e-2
    assert scaled_err(got, ref32) < 2e-2 and rel_rms(got, ref32) < 1.5e-2
    # and the device is as close to fp32 as the bf16-storage oracle is (25 % slack)
    assert np.abs(got - ref32).max() < 1.25 * np.abs(ref - ref32).max()
