"""MLP forward + backward + Adam through the host-side tape, against the CPU oracle; and
two data-parallel ranks whose weights must stay bit-identical.

Tolerances: loss within 1e-3 relative; bf16 gradients within max-abs 2e-2 of the oracle's
gradient scaled to O(1) (gradients are ~1e-5, so the comparison is made on g / max|g|);
the Adam kernel itself, fed the same gradient, matches the oracle to fp32 rounding."""
import numpy as np
import pytest

import oracle
from oracle import mlp
from util import SEED, bf16_normal

pytestmark = pytest.mark.gpu
WIDTH, BATCH, LAYERS = 256, 128, 4


def test_adam_kernel_matches_oracle(ctx):
    n = 4096
    w = oracle.normal((n,), SEED + 80)
    g, gb = bf16_normal((n,), SEED + 81, 1e-3)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    dw, dm, dv, dg = ctx.upload(w), ctx.upload(m), ctx.upload(v), ctx.upload(gb)
    dwb = ctx.empty((n,))
    rw, rm, rv = w.copy(), m.copy(), v.copy()
    for step in (1, 2, 3):
        ctx.adam_step(dw, dm, dv, dg, dwb, step, grad_scale=0.5)
        oracle.adam(rw, rm, rv, g * np.float32(0.5), step=step)
    assert np.allclose(ctx.download(dw), rw, rtol=0, atol=2e-6)
    assert np.allclose(ctx.download(dm), rm, rtol=1e-5, atol=1e-9)
    assert np.allclose(ctx.download(dv), rv, rtol=1e-5, atol=1e-12)
    assert np.array_equal(ctx.download(dwb), oracle.to_bf16_bits(ctx.download(dw)))


def test_mse_kernel(ctx):
    y, yb = bf16_normal((1000, 37), SEED + 82)
    t, tb = bf16_normal((1000, 37), SEED + 83)
    loss, dy = ctx.mse(ctx.upload(yb), ctx.upload(tb))
    assert abs(float(ctx.download(loss)[0]) - oracle.mse(y, t)) < 1e-5
    ref = (y - t) * np.float32(2.0 / y.size)
    got = oracle.from_bf16_bits(ctx.download(dy))
    assert np.max(np.abs(got - ref)) <= 2.0 ** -8 * np.max(np.abs(ref))


def _run_steps(ctx, world=1, rank=0, n_steps=2, trainer_kwargs=None):
    from habu_b200.autograd import MlpTrainer
    ws = mlp.make_weights(WIDTH, LAYERS)
    tr = MlpTrainer(ctx, WIDTH, BATCH, LAYERS, ws, world=world, **(trainer_kwargs or {}))
    x, y = mlp.make_batch(BATCH, WIDTH, rank)
    dx, dy = ctx.upload(oracle.to_bf16_bits(x)), ctx.upload(oracle.to_bf16_bits(y))
    losses = []
    for _ in range(n_steps):
        tr.step(dx, dy)
        ctx.sync()
        losses.append(float(ctx.download(tr.loss)[0]))
    return tr, losses


def test_training_step_matches_oracle(ctx):
    tr, losses = _run_steps(ctx, n_steps=1)
    ws = mlp.make_weights(WIDTH, LAYERS)
    wb = [oracle.round_bf16(w.copy()) for w in ws]
    x, y = mlp.make_batch(BATCH, WIDTH)
    loss, grads = mlp.forward_backward(wb, x, y)
    assert abs(losses[0] - loss) / loss < 1e-3
    for i in range(LAYERS):
        got = oracle.from_bf16_bits(ctx.download(tr.grads[i]))
        scale = np.max(np.abs(grads[i]))
        assert np.max(np.abs(got - grads[i])) / scale < 2e-2, i
    # Adam with the device's own gradients reproduces the device's weights
    m = [np.zeros_like(w) for w in ws]
    v = [np.zeros_like(w) for w in ws]
    dev_grads = [oracle.from_bf16_bits(ctx.download(g)) for g in tr.grads]
    mlp.adam_update(ws, m, v, dev_grads, step=1)
    for i in range(LAYERS):
        assert np.allclose(ctx.download(tr.w32[i]), ws[i], rtol=0, atol=2e-6), i


def test_loss_decreases_over_steps(ctx):
    _, losses = _run_steps(ctx, n_steps=8)
    assert losses[-1] < losses[0]


def test_checkpoint_resume_reproduces_the_next_step_bit_for_bit(ctx, tmp_path):
    """save -> load into a fresh trainer -> one more step: weights, moments and loss equal
    those of the trainer that kept running."""
    from habu_b200.autograd import MlpTrainer
    tr, _ = _run_steps(ctx, n_steps=2)
    path = str(tmp_path / "mlp.ckpt")
    tr.save(path)
    x, y = mlp.make_batch(BATCH, WIDTH)
    dx, dy = ctx.upload(oracle.to_bf16_bits(x)), ctx.upload(oracle.to_bf16_bits(y))
    tr.step(dx, dy)
    ctx.sync()
    other = MlpTrainer(ctx, WIDTH, BATCH, LAYERS, [np.zeros((WIDTH, WIDTH), np.float32)] * LAYERS)
    other.load(path)
    assert other.step_no == 2
    other.step(dx, dy)
    ctx.sync()
    assert ctx.download(other.loss).tobytes() == ctx.download(tr.loss).tobytes()
    for i in range(LAYERS):
        for a, b in ((tr.w32[i], other.w32[i]), (tr.m[i], other.m[i]), (tr.v[i], other.v[i]), (tr.wb[i], other.wb[i])):
            assert ctx.download(a).tobytes() == ctx.download(b).tobytes(), i
    with open(path, "r+b") as f:          # a truncated file is refused
        f.truncate(1000)
    with pytest.raises(ValueError):
        other.load(path)


@pytest.mark.timeout(900)
def test_full_size_step_matches_oracle():
    """The benchmark's own configuration: 4 layers of width 8192, batch 4096, one forward +
    backward + Adam step against the CPU oracle (about 6 TFLOP on the host cores)."""
    import habu_b200 as hb
    from habu_b200.autograd import MlpTrainer
    width, batch, layers = 8192, 4096, 4
    oracle.use_all_cores()
    ctx = hb.Context(0)
    try:
        ws = mlp.make_weights(width, layers)
        tr = MlpTrainer(ctx, width, batch, layers, ws)
        x, y = mlp.make_batch(batch, width)
        dx, dy = ctx.upload(oracle.to_bf16_bits(x)), ctx.upload(oracle.to_bf16_bits(y))
        tr.step(dx, dy)
        ctx.sync()
        got_loss = float(ctx.download(tr.loss)[0])
        wb = [oracle.round_bf16(w.copy()) for w in ws]
        loss, grads = mlp.forward_backward(wb, x, y)
        del wb
        assert abs(got_loss - loss) / loss < 1e-3, (got_loss, loss)
        for i in range(layers):
            got = oracle.from_bf16_bits(ctx.download(tr.grads[i]))
            scale = float(np.max(np.abs(grads[i])))
            err = float(np.max(np.abs(got - grads[i]))) / scale
            assert err < 2e-2, (i, err)          # bf16 gradients, compared on g / max|g|
            # Adam fed the device's own gradient reproduces the device's weights to fp32 rounding
            m, v = np.zeros_like(ws[i]), np.zeros_like(ws[i])
            mlp.adam_update([ws[i]], [m], [v], [got], step=1)
            assert np.allclose(ctx.download(tr.w32[i]), ws[i], rtol=0, atol=2e-6), i
            assert np.array_equal(ctx.download(tr.wb[i]), oracle.to_bf16_bits(ctx.download(tr.w32[i]))), i
            grads[i] = None
    finally:
        ctx.close()


def _dp_rank(rank, world):
    import torch.distributed as dist

    import habu_b200 as hb
    from habu_b200.autograd import MlpTrainer
    from mp_util import RankGuard, init_group
    init_group("gloo", rank, world)
    guard = RankGuard()
    ctx = None
    with guard:
        ctx = hb.Context(rank)
        ctx.comm_set_wait_limit(1 << 22)
        ids = [hb.Context.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        ctx.comm_init_rank(world, rank, ids[0])
        nbytes = MlpTrainer.grad_bytes(WIDTH, LAYERS)
        ptr, handle = ctx.p2p_alloc(nbytes)
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        ctx.p2p_attach(world, rank, handles, nbytes)
    if guard.agree():
        with guard:
            tr, losses = _run_steps(ctx, world, rank, n_steps=1, trainer_kwargs={"grads_base_ptr": ptr})
            # the summed gradient / world equals the oracle's gradient over the concatenated batch
            ws = [oracle.round_bf16(w.copy()) for w in mlp.make_weights(WIDTH, LAYERS)]
            xs, ys = zip(*[mlp.make_batch(BATCH, WIDTH, r) for r in range(world)])
            _, grads_all = mlp.forward_backward(ws, np.concatenate(xs), np.concatenate(ys))
            for i in range(LAYERS):
                got = oracle.from_bf16_bits(ctx.download(tr.grads[i])) / world
                assert np.max(np.abs(got - grads_all[i])) / np.max(np.abs(grads_all[i])) < 2e-2, i
    if guard.agree():
        with guard:
            x, y = mlp.make_batch(BATCH, WIDTH, rank)
            dx, dy = ctx.upload(oracle.to_bf16_bits(x)), ctx.upload(oracle.to_bf16_bits(y))
            for _ in range(2):
                tr.step(dx, dy)
            ctx.sync()
            mine = b"".join(ctx.download(w).tobytes() for w in tr.w32)
    if guard.agree():
        with guard:
            blobs = [None] * world
            dist.all_gather_object(blobs, mine)
            assert all(b == blobs[0] for b in blobs), "weights diverged across data-parallel ranks"
    if ctx is not None:
        ctx.sync() if guard.error is None and not guard.peer_failed else None
    dist.barrier()                 # nobody unmaps its buffer while a peer's kernel may still read it
    if ctx is not None:
        ctx.close()
    dist.destroy_process_group()
    guard.reraise()


def test_two_data_parallel_ranks_stay_identical():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    from mp_util import run_ranks
    run_ranks(_dp_rank, 2)
