"""Golden fixtures (`tests/golden/oracle_small.npz`, written by `tests/golden/make_golden.py`).

They are outputs of this repository's own CPU oracle on small seeded cases -- the reference
project has nothing to take golden vectors from -- and serve two purposes: the CPU suite
checks that today's oracle still reproduces them (so a change to the oracle or to the
seeded generators cannot slip through unnoticed), and the GPU suite checks the device
results against the stored values, independent of the oracle library being rebuilt."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

import oracle  # noqa: E402
from make_golden import cases  # noqa: E402
from util import bf16_close, max_abs, max_rel  # noqa: E402

GOLDEN = np.load(os.path.join(HERE, "golden", "oracle_small.npz"))


def test_fixture_file_covers_every_case():
    assert sorted(GOLDEN.files) == sorted(cases())


def test_oracle_reproduces_the_golden_outputs():
    for name, (_, expected) in cases().items():
        assert GOLDEN[name].shape == expected.shape, name
        # same code, same inputs: equal up to the summation order OpenMP may choose
        assert max_abs(GOLDEN[name], expected) < 1e-6, name


@pytest.mark.gpu
def test_device_results_match_the_golden_outputs(ctx):
    import habu_b200 as hb
    c = cases()
    bits = oracle.to_bf16_bits
    back = oracle.from_bf16_bits

    i, _ = c["gemm_bf16_128x256x64"]
    got = back(ctx.download(ctx.matmul(ctx.upload(bits(i["A"])), ctx.upload(bits(i["Bt"])).T)))
    assert max_abs(got, GOLDEN["gemm_bf16_128x256x64"]) < 2e-2

    i, _ = c["gemm_f32_100x37x50"]
    got = ctx.download(ctx.matmul(ctx.upload(i["A"]), ctx.upload(i["B"])))
    assert max_rel(got, GOLDEN["gemm_f32_100x37x50"]) < 1e-4

    i, _ = c["attention_causal_gqa_s136"]
    got = back(ctx.download(ctx.attention(ctx.upload(bits(i["Q"])), ctx.upload(bits(i["K"])), ctx.upload(bits(i["V"])))))
    assert max_abs(got, GOLDEN["attention_causal_gqa_s136"]) < 2e-2

    i, _ = c["rmsnorm_24x256"]
    got = back(ctx.download(ctx.rmsnorm(ctx.upload(bits(i["x"])), ctx.upload(bits(i["g"])), eps=1e-5)))
    assert bf16_close(got, GOLDEN["rmsnorm_24x256"]) < 0
    ctx.sync()
