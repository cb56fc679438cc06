"""Data-parallel contract of the MLP training step on CPU ranks (gloo): each rank
differentiates the mean-squared error of its own batch, gradients are summed across ranks
and Adam applies them scaled by 1/world -- which must equal one step on the concatenated
batch.  The device trainer (`habu_b200.autograd.MlpTrainer`) follows the same convention;
this test pins the convention itself with the oracle, no GPU involved."""
import numpy as np

from mp_util import init_group, run_ranks

WIDTH, BATCH, LAYERS = 64, 32, 3


def _rank(rank, world):
    import torch
    import torch.distributed as dist

    import oracle
    from oracle import mlp
    init_group("gloo", rank, world)
    ws = mlp.make_weights(WIDTH, LAYERS)
    wb = [oracle.round_bf16(w.copy()) for w in ws]        # bf16 working copy; round_bf16 works in place
    x, y = mlp.make_batch(BATCH, WIDTH, rank)
    loss, grads = mlp.forward_backward(wb, x, y, round_bf16=False)
    summed = []
    for g in grads:
        t = torch.from_numpy(np.ascontiguousarray(g))
        dist.all_reduce(t)                               # sum, like the device collective
        summed.append(t.numpy())
    m = [np.zeros_like(w) for w in ws]
    v = [np.zeros_like(w) for w in ws]
    mlp.adam_update(ws, m, v, summed, step=1, grad_scale=1.0 / world)

    # the same step on the concatenated batch, computed by every rank on its own
    xs, ys = zip(*[mlp.make_batch(BATCH, WIDTH, r) for r in range(world)])
    ws_ref = mlp.make_weights(WIDTH, LAYERS)
    loss_all, grads_all = mlp.forward_backward(wb, np.concatenate(xs), np.concatenate(ys), round_bf16=False)
    for g, ga in zip(summed, grads_all):
        assert np.allclose(g / world, ga, rtol=1e-4, atol=1e-7), float(np.abs(g / world - ga).max())
    m2 = [np.zeros_like(w) for w in ws_ref]
    v2 = [np.zeros_like(w) for w in ws_ref]
    mlp.adam_update(ws_ref, m2, v2, grads_all, step=1)
    for w, wr in zip(ws, ws_ref):
        # Adam's first step moves every weight by about lr; the two routes agree far below that
        assert np.abs(w - wr).max() < 2e-5

    # the mean of the per-rank losses is the loss of the concatenated batch
    t = torch.tensor([loss], dtype=torch.float64)
    dist.all_reduce(t)
    assert abs(t.item() / world - loss_all) < 1e-6 * max(1.0, abs(loss_all))

    # replicas stay bit-identical: every rank applied the same summed gradient
    gathered = [None] * world
    dist.all_gather_object(gathered, b"".join(w.tobytes() for w in ws))
    assert all(g == gathered[0] for g in gathered)
    dist.destroy_process_group()


def test_two_cpu_ranks_sum_gradients_like_one_big_batch():
    run_ranks(_rank, 2, timeout=240)
