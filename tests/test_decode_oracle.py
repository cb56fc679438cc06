"""The oracle's generation step against its own prefill forward (CPU only): the step for
token t must reproduce row t of the forward over the same sequence -- to fp32 rounding in the
fp32 mode, within one bf16 rounding in the bf16-storage mode.  This ties `decode_step`, which
the GPU decode tests are checked against, to `forward`, which everything else is."""
import numpy as np

from habu_b200.tp import DecoderConfig
from oracle import decoder
from util import bf16_close


def test_decode_step_reproduces_the_rows_of_the_prefill_forward():
    cfg = DecoderConfig(d_model=256, n_q_heads=4, n_kv_heads=2, head_dim=128, ffn_hidden=512, n_layers=2, batch=2, seq=20)
    layers = [decoder.make_layer(cfg, i) for i in range(cfg.n_layers)]
    x0 = decoder.make_input(cfg)
    xs = x0.reshape(cfg.batch, cfg.seq, -1)
    for bf16 in (False, True):
        ref = decoder.forward(cfg, x0, layers, round_bf16=bf16).reshape(cfg.batch, cfg.seq, -1)
        cache = decoder.new_cache(cfg, cfg.batch, cfg.seq)
        for t in range(cfg.seq):
            y = decoder.decode_step(cfg, np.ascontiguousarray(xs[:, t]), layers, cache, t, round_bf16=bf16)
            if bf16:
                assert bf16_close(y, ref[:, t]) < 0, t
            else:
                assert np.abs(y - ref[:, t]).max() < 1e-5, t
