"""Failure detection without a GPU fault: a cross-GPU flag wait that runs out.

One process, one GPU.  The context is given a two-rank "external" symmetric mapping whose
second rank is a second local buffer that no kernel ever writes flags into -- a peer that
never arrives.  With the wait limit set to a few thousand polls the allreduce kernel gives
up at its first handshake, records HB_ERR_TIMEOUT (kernel tag 3 = allreduce, detail 0 = the
opening handshake) and returns without touching the payload; hb_sync reports it, clears the
status, and the same context then runs a matmul correctly.  Nothing traps, faults or hangs.
"""
import numpy as np
import pytest

import oracle
from util import SEED, bf16_normal, max_abs

pytestmark = pytest.mark.gpu


def test_allreduce_wait_runs_out_and_the_context_stays_usable():
    import habu_b200 as hb
    from habu_b200.model_ir import HabuError
    ctx = hb.Context(0)
    try:
        count = 1 << 16
        flag = hb.Context.p2p_flag_bytes()
        mine = ctx.upload(np.zeros(count * 2 + flag, np.uint8).view(np.uint16))     # payload, then zeroed flags
        absent = ctx.upload(np.zeros(count * 2 + flag, np.uint8).view(np.uint16))   # the rank that never arrives
        ctx.p2p_attach_external(2, 0, [mine.ptr, absent.ptr], None, count * 2)
        ctx.comm_set_wait_limit(4096)
        x, xb = bf16_normal((count,), SEED + 401)
        import ctypes as C
        from habu_b200 import model_ir
        ctx._check(model_ir._lib.hb_upload(ctx._h, mine.ptr, xb.ctypes.data_as(C.c_void_p), xb.nbytes))
        ctx.sync()
        data = ctx.wrap(mine.ptr, (count,))
        for attempt in range(2):                        # the status clears, so the second time-out is reported too
            ctx.all_reduce(data, hb.HB_AR_P2P)
            with pytest.raises(HabuError) as err:
                ctx.sync()
            assert err.value.status == 6, err.value     # HB_ERR_TIMEOUT
            assert "kernel tag 3" in str(err.value) and "detail 0" in str(err.value)
        ctx.sync()                                      # status was cleared: no stale error
        # the kernel gave up before its data phase: the payload is untouched
        got = np.empty(count, np.uint16)
        ctx._check(model_ir._lib.hb_download(ctx._h, got.ctypes.data_as(C.c_void_p), mine.ptr, got.nbytes))
        ctx.sync()
        assert np.array_equal(got, xb)
        # the context is still usable
        A, Ab = bf16_normal((256, 512), SEED + 402, 512 ** -0.5)
        Bt, Btb = bf16_normal((384, 512), SEED + 403)
        dC = ctx.matmul(ctx.upload(Ab), ctx.upload(Btb).T)
        ctx.sync()
        assert max_abs(oracle.from_bf16_bits(ctx.download(dC)), oracle.gemm(A, Bt.T)) < 2e-2
        with pytest.raises(HabuError):
            ctx.comm_set_wait_limit(0)
    finally:
        ctx.close()
