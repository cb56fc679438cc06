#!/usr/bin/env python
"""Benchmark of the dense hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemm|skinny|attention]
                    [--impl ours|reference]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  The
default workload is the bf16 GEMM at M=N=K=8192 (A row-major, B column-major, fp32
accumulate, bf16 output).  Rank 0 prints ONE JSON line:

  value         whole-job TFLOP/s with operands resident in HBM, CUDA-event timed on the
                launching stream, max over ranks (N>1: independent replicas, one per GPU);
  e2e           the same metric through the host-buffer C-ABI call (pinned host buffers,
                host->device and device->host copies inside the timed region);
  roofline      dominant kernel: algorithmic flop per launch / measured launch duration,
                against the measured cuBLAS bf16 peak in MEASURED_PEAKS.json;
  cpu_baseline  the CPU oracle timed on the host cores on a bounded sample (rank 0, N=1).

``--impl reference`` times the reference arm: the reference project has no implementation
of this path, so the CPU oracle (a port, all host threads) stands in for it.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

SEED = 0x48414255
NVSMI_Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
           "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu capture
# (profiles/), scaled to the full launch; None where not captured.
NCU_TRAFFIC_BYTES = {"gemm": 1.128998e9 + 127.475712e6, "skinny": 134.593280e6 + 4.446208e6,
                     "attention": 805.502464e6 + 257.930496e6}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "hbm": d["hbm_gbs"], "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU during the timed region."""

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={NVSMI_Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v == "Active"})
        pw = [float(r[3]) for r in self.rows if len(r) >= 9 and r[3].replace(".", "").isdigit()]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": reasons}


# --------------------------------------------------------------------------- workloads
class GemmWorkload:
    """bf16 GEMM C = A.B, A [M,K] row-major, B column-major, N(0,1)/sqrt(K) entries."""
    bound = "tensor"
    kernel = "hb_gemm_bf16_pair_kernel"     # the autotune cache picks the CTA-pair tile for the large shapes

    def __init__(self, name, M, N, K):
        self.name, self.M, self.N, self.K = name, M, N, K
        self.flop = 2.0 * M * N * K
        self.bytes = 2.0 * (M * K + N * K + M * N)
        self.metric, self.unit = "bf16_gemm_tflops", "TFLOP/s"
        self.desc = f"bf16 GEMM M={M} N={N} K={K}, A row-major, B column-major, fp32 accumulate, bf16 out"
        if name == "skinny":
            self.bound = "hbm"
            self.kernel = "hb_gemm_skinny_kernel"

    def host_inputs(self, rank):
        import oracle
        s = SEED + 1000 * rank
        A = oracle.to_bf16_bits(oracle.normal((self.M, self.K), s + 1, 0.0, self.K ** -0.5))
        Bt = oracle.to_bf16_bits(oracle.normal((self.N, self.K), s + 2, 0.0, self.K ** -0.5))
        return A, Bt

    def setup(self, ctx, rank, pinned):
        A, Bt = self.host_inputs(rank)
        self.hA, self.hB = pinned(A), pinned(Bt)
        self.hC = pinned(np.empty((self.M, self.N), np.uint16))
        self.h2d, self.d2h = A.nbytes + Bt.nbytes, self.hC.nbytes
        # Timing hygiene: when A + B + C do not exceed the 126 MB L2 by a wide margin, the
        # steps rotate over enough separate copies of the operands that every launch reads
        # cold data (the copies together are >= 2.5x L2).
        self.flush = None
        copies = 1 if self.bytes >= 2 * 126e6 else int(np.ceil(2.5 * 126e6 / self.bytes))
        self.sets = [(ctx.upload(A), ctx.upload(Bt), ctx.empty((self.M, self.N))) for _ in range(copies)]
        self.dA, self.dB, self.dC = self.sets[0]
        self.turn = 0
        self.flush_note = ("inputs larger than L2 (A+B+C = %.0f MB)" % (self.bytes / 1e6) if copies == 1 else
                           "steps rotate over %d copies of A, B, C (%.0f MB in total, larger than L2)"
                           % (copies, copies * self.bytes / 1e6))

    def step(self, ctx):
        dA, dB, dC = self.sets[self.turn % len(self.sets)]
        self.turn += 1
        ctx.matmul(dA, dB.T, out=dC)

    def step_e2e(self, ctx):
        import ctypes as C
        from habu_b200 import model_ir
        st = model_ir._lib.hb_matmul_host(ctx._h, self.hA.ctypes.data_as(C.c_void_p), self.hB.ctypes.data_as(C.c_void_p),
                                          self.hC.ctypes.data_as(C.c_void_p), self.M, self.N, self.K, 1)
        ctx._check(st)

    def cpu_sample(self, max_rows=4096):
        """Bounded CPU sample: the first `rows` rows of the same GEMM on the oracle."""
        import oracle
        rows = min(self.M, max_rows)
        A = oracle.round_bf16(oracle.normal((rows, self.K), SEED + 1, 0.0, self.K ** -0.5))
        Bt = oracle.round_bf16(oracle.normal((self.N, self.K), SEED + 2, 0.0, self.K ** -0.5))
        t0 = time.perf_counter()
        oracle.gemm(A, Bt.T)
        dt = time.perf_counter() - t0
        return 2.0 * rows * self.N * self.K / dt / 1e12, f"first {rows} of {self.M} rows of C (oracle GEMM, fp32)"


class AttentionWorkload:
    """Fused causal self-attention forward, bf16: Q/K/V [B,S,H,128] ~ N(0,1), scale 1/sqrt(128)."""
    bound = "tensor"
    kernel = "hb_attention_fwd_kernel"
    flush = None

    def __init__(self, name, B, S, H, D=128):
        self.name, self.B, self.S, self.H, self.D = name, B, S, H, D
        self.flop = 4.0 * B * H * S * S * D / 2          # conventional causal count
        self.bytes = 4.0 * B * S * H * D * 2
        self.metric, self.unit = "bf16_causal_attention_tflops", "TFLOP/s"
        self.desc = (f"fused causal self-attention forward bf16: batch {B}, {H} heads, seq {S}, head_dim {D}, "
                     "Q/K/V N(0,1), scale 1/sqrt(128), layout [batch, seq, heads, head_dim]")
        self.flush_note = "inputs larger than L2 (Q+K+V+O = %.0f MB)" % (self.bytes / 1e6)

    def setup(self, ctx, rank, pinned):
        import oracle
        shape = (self.B, self.S, self.H, self.D)
        s = SEED + 1000 * rank
        hs = [oracle.to_bf16_bits(oracle.normal(shape, s + 10 + i)) for i in range(3)]
        self.hQ, self.hK, self.hV = (pinned(h) for h in hs)
        self.hO = pinned(np.empty(shape, np.uint16))
        self.dQ, self.dK, self.dV = (ctx.upload(h) for h in hs)
        self.dO = ctx.empty(shape)
        self.h2d, self.d2h = 3 * hs[0].nbytes, hs[0].nbytes

    def step(self, ctx):
        ctx.attention(self.dQ, self.dK, self.dV, out=self.dO, causal=True)

    def step_e2e(self, ctx):
        import ctypes as C
        from habu_b200 import model_ir
        vp = lambda a: a.ctypes.data_as(C.c_void_p)
        ctx._check(model_ir._lib.hb_attention_host(ctx._h, vp(self.hQ), vp(self.hK), vp(self.hV), vp(self.hO), self.B,
                                                   self.S, self.H, self.H, self.D, 1, self.D ** -0.5))

    def cpu_sample(self, max_rows=None):
        """Bounded CPU sample: full causal attention of 4 (batch, head) pairs on the oracle."""
        import oracle
        heads = 4 if max_rows is None else 1
        shape = (1, self.S, heads, self.D)
        Q, K, V = (oracle.round_bf16(oracle.normal(shape, SEED + 10 + i)) for i in range(3))
        t0 = time.perf_counter()
        oracle.attention(Q, K, V, causal=True)
        dt = time.perf_counter() - t0
        return (4.0 * heads * self.S * self.S * self.D / 2 / dt / 1e12,
                f"{heads} of {self.B * self.H} (batch, head) pairs at seq {self.S} (oracle attention, fp32)")


def attach_symmetric(ctx, rank, world, dist, nbytes):
    """Gives the context a peer-mapped buffer of `nbytes` for its collectives and returns its
    local address.  HB_COMM=nvls (default): torch's symmetric-memory allocator supplies the
    buffer and its NVSwitch multicast mapping (plumbing only; the reduction kernels are the
    library's); falls back to HB_COMM=p2p (the library's own cudaIpc mapping, no multicast)
    when no multicast mapping is available."""
    mode = os.environ.get("HB_COMM", "nvls")
    if mode == "nvls":
        try:
            import torch
            import torch.distributed._symmetric_memory as symm
            payload = (nbytes + 255) // 256 * 256
            buf = symm.empty(payload + ctx.p2p_flag_bytes(), dtype=torch.uint8, device=f"cuda:{torch.cuda.current_device()}")
            buf.zero_()
            hdl = symm.rendezvous(buf, dist.group.WORLD)
            torch.cuda.synchronize()
            dist.barrier()
            if hdl.multicast_ptr:
                ctx.p2p_attach_external(world, rank, list(hdl.buffer_ptrs), hdl.multicast_ptr, nbytes)
                attach_symmetric.keep.append((buf, hdl))
                return hdl.buffer_ptrs[rank], "nvls"
        except Exception as e:   # plumbing unavailable: use the library's own mapping
            if rank == 0:
                print(f"symmetric-memory plumbing unavailable ({e}); using cudaIpc peer mapping", file=sys.stderr)
    ptr, handle = ctx.p2p_alloc(nbytes)
    handles = [None] * world
    dist.all_gather_object(handles, handle)
    ctx.p2p_attach(world, rank, handles, nbytes)
    return ptr, "p2p"


attach_symmetric.keep = []


class DecoderWorkload:
    """Llama-style decoder block forward x2 layers, bf16, tensor-parallel over all ranks:
    d_model 4096, 32 query / 8 KV heads, head_dim 128, SwiGLU hidden 14336, batch 4 x seq 2048."""
    bound = "tensor"
    kernel = "hb_gemm_bf16_pair_kernel"     # dominant kernel of the step (projections and FFN products)
    flush = None
    scaling = "strong"
    collective = True

    def __init__(self, name="decoder"):
        from habu_b200.tp import DecoderConfig
        self.name, self.cfg = name, DecoderConfig()
        self.flop = self.cfg.flops()
        self.tokens = self.cfg.tokens
        self.metric, self.unit = "decoder_tokens_per_s", "tokens/s"
        self.desc = ("Llama-style decoder block forward x2 layers bf16: d_model 4096, 32 q / 8 kv heads, head_dim 128, "
                     "SwiGLU 14336, RMSNorm eps 1e-5, RoPE base 10000, batch 4 x seq 2048, weights N(0,0.02), "
                     "embeddings N(0,1); Megatron tensor parallel, allreduce after attention-out and FFN-down")
        self.flush_note = "weights + activations per step exceed L2 (weights alone 872 MB / TP)"

    def setup(self, ctx, rank, pinned, world=1, dist=None):
        import oracle
        from habu_b200 import HB_AR_AUTO
        from habu_b200.tp import DecoderGraph, shard_layer
        from oracle import decoder
        cfg = self.cfg
        layers = []
        for i in range(cfg.n_layers):
            full = decoder.make_layer(cfg, i)
            layers.append({k: oracle.to_bf16_bits(v) for k, v in shard_layer(full, cfg, world, rank).items()})
            del full
        # micro-batches whose allreduce overlaps the next chunk's GEMMs (only useful with peers)
        self.chunks = int(os.environ.get("HB_DECODER_CHUNKS", "1"))
        # fused reduce-scatter + residual + RMSNorm + all-gather nodes instead of allreduce + replicated norms
        self.fused = os.environ.get("HB_DECODER_FUSED", "1") == "1" and world > 1 and self.chunks == 1
        self.dg = DecoderGraph(ctx, cfg, world, rank, layers, HB_AR_AUTO, self.chunks, fused=self.fused)
        _, sym = self.dg.plan()
        if world > 1:
            ids = [ctx.comm_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            ctx.comm_init_rank(world, rank, ids[0])
            _, self.comm = attach_symmetric(ctx, rank, world, dist, sym)
            self.dg.plan()
        x0 = oracle.to_bf16_bits(decoder.make_input(cfg))
        self.hX = pinned(x0)
        self.hO = pinned(np.empty_like(x0))
        self._copy(ctx, self.dg.x0.ptr, self.hX, up=True)
        ctx.sync()
        self.h2d, self.d2h = x0.nbytes, x0.nbytes
        self.world = world

    @staticmethod
    def _copy(ctx, dev_ptr, host, up):
        import ctypes as C
        from habu_b200 import model_ir
        f = model_ir._lib.hb_upload if up else model_ir._lib.hb_download
        a, b = (C.c_void_p(dev_ptr), host.ctypes.data_as(C.c_void_p))
        ctx._check(f(ctx._h, a, b, host.nbytes) if up else f(ctx._h, b, a, host.nbytes))

    def step(self, ctx):
        self.dg.run()

    def step_e2e(self, ctx):
        self._copy(ctx, self.dg.x0.ptr, self.hX, up=True)
        self.dg.run()
        self._copy(ctx, self.dg.out.ptr, self.hO, up=False)
        ctx.sync()

    def value(self, ms, world):
        return self.tokens / (ms * 1e-3)

    def cpu_sample(self, max_rows=None):
        """Bounded CPU sample: the same block at batch 1 x seq 256 on the oracle (fp32)."""
        from dataclasses import replace
        from oracle import decoder
        cfg = replace(self.cfg, batch=1, seq=256 if max_rows is None else 128, n_layers=1)
        layers = [decoder.make_layer(cfg, 0)]
        x0 = decoder.make_input(cfg)
        t0 = time.perf_counter()
        decoder.forward(cfg, x0, layers, round_bf16=False)
        dt = time.perf_counter() - t0
        return cfg.tokens / dt * (1.0 / self.cfg.n_layers), (
            f"1 of {self.cfg.n_layers} layers at batch 1 x seq {cfg.seq} (oracle decoder, fp32), scaled to tokens/s of "
            f"the {self.cfg.n_layers}-layer block")


class MlpWorkload:
    """4-layer MLP forward + backward + Adam, width 8192, GELU, batch 4096 per GPU, MSE; bf16
    activations / gradients, fp32 master weights and moments; data-parallel gradient allreduce."""
    bound = "tensor"
    kernel = "hb_gemm_bf16_pair_kernel"     # dominant kernel of the step (forward and both backward products)
    flush = None
    scaling = "weak"
    collective = True

    def __init__(self, name="mlp", width=8192, batch=4096, layers=4):
        self.name, self.width, self.batch, self.layers = name, width, batch, layers
        fwd = layers * 2.0 * batch * width * width
        self.flop = fwd + fwd + (layers - 1) * 2.0 * batch * width * width   # fwd + dW + dX (no dX for layer 0)
        self.metric, self.unit = "mlp_train_samples_per_s", "samples/s"
        self.desc = (f"{layers}-layer MLP fwd+bwd+Adam: width {width}, GELU, batch {batch} per GPU, MSE, Adam lr 1e-3 "
                     "b=(0.9,0.999) eps 1e-8, bf16 activations and gradients, fp32 master weights and moments; "
                     "data-parallel bf16 gradient allreduce")
        self.flush_note = "weights, moments and activations per step (>4 GB) exceed L2"

    def setup(self, ctx, rank, pinned, world=1, dist=None):
        import oracle
        from habu_b200.autograd import MlpTrainer
        from oracle import mlp
        ws = mlp.make_weights(self.width, self.layers)
        base = None
        if world > 1:
            ids = [ctx.comm_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            ctx.comm_init_rank(world, rank, ids[0])
            nbytes = MlpTrainer.grad_bytes(self.width, self.layers)
            base, self.comm = attach_symmetric(ctx, rank, world, dist, nbytes)
        self.tr = MlpTrainer(ctx, self.width, self.batch, self.layers, ws, world=world, grads_base_ptr=base)
        del ws
        x, y = mlp.make_batch(self.batch, self.width, rank)
        xb, yb = oracle.to_bf16_bits(x), oracle.to_bf16_bits(y)
        self.hX, self.hY = pinned(xb), pinned(yb)
        self.hL = pinned(np.zeros(1, np.float32))
        self.dX, self.dY = ctx.upload(xb), ctx.upload(yb)
        self.h2d, self.d2h = xb.nbytes + yb.nbytes, 4
        self.world = world

    def step(self, ctx):
        self.tr.step(self.dX, self.dY)

    def step_e2e(self, ctx):
        DecoderWorkload._copy(ctx, self.dX.ptr, self.hX, up=True)
        DecoderWorkload._copy(ctx, self.dY.ptr, self.hY, up=True)
        self.tr.step(self.dX, self.dY)
        DecoderWorkload._copy(ctx, self.tr.loss.ptr, self.hL, up=False)
        ctx.sync()

    def value(self, ms, world):
        return self.batch * world / (ms * 1e-3)

    def cpu_sample(self, max_rows=None):
        """Bounded CPU sample: one fwd+bwd+Adam step at width 1024, batch 512 on the oracle."""
        from oracle import mlp
        width, batch = (1024, 512) if max_rows is None else (512, 256)
        ws = mlp.make_weights(width, self.layers)
        x, y = mlp.make_batch(batch, width)
        m = [np.zeros_like(w) for w in ws]
        v = [np.zeros_like(w) for w in ws]
        t0 = time.perf_counter()
        _, grads = mlp.forward_backward(ws, x, y, round_bf16=False)
        mlp.adam_update(ws, m, v, grads, 1)
        dt = time.perf_counter() - t0
        scale = (batch * width * width) / (self.batch * self.width * self.width)   # flop ratio sample / full step
        return self.batch * scale / dt, (f"one step at width {width}, batch {batch} (oracle, fp32), scaled by the flop "
                                         f"ratio to samples/s of the width-{self.width} model")


WORKLOADS = {
    "mlp": lambda: MlpWorkload(),
    "attention": lambda: AttentionWorkload("attention", 8, 4096, 32),
    "decoder": lambda: DecoderWorkload(),
    "gemm": lambda: GemmWorkload("gemm", 8192, 8192, 8192),
    "gemm4096": lambda: GemmWorkload("gemm4096", 4096, 4096, 4096),
    "gemm1024": lambda: GemmWorkload("gemm1024", 1024, 1024, 1024),
    "skinny": lambda: GemmWorkload("skinny", 16, 8192, 8192),
}


def run_reference(args, rank, world):
    """Reference arm: the CPU oracle (port) on all host threads, bounded sample per step."""
    if rank != 0:
        return
    import oracle
    oracle.use_all_cores()
    wl = WORKLOADS[args.workload]()
    vals, times = [], []
    sample = ""
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        v, sample = wl.cpu_sample(max_rows=1024)
        if i >= args.warmup:
            vals.append(v)
            times.append((time.perf_counter() - t0) * 1e3)
    v = float(np.mean(vals))
    line = {"impl": "reference", "metric": wl.metric, "value": v, "unit": wl.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(times)), "higher_is_better": True,
            "scaling": getattr(wl, "scaling", "weak"), "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl.desc, "parallelism": "host CPU threads",
                       "step": "one bounded sample of the workload: " + sample},
            "cpu_baseline": {"value": v, "unit": wl.unit, "cores": oracle.num_threads(), "kind": "port",
                             "sample": sample + "; the reference project has no implementation of this path"},
            "e2e": {"value": v, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="gemm", choices=sorted(WORKLOADS))
    ap.add_argument("--extras", default="attention,decoder",
                    help="comma-separated workloads also measured (device-resident leg only) and reported under 'extras'")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    import habu_b200 as hb

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    stream = torch.cuda.Stream()
    pk = peaks()

    def pinned(a: np.ndarray) -> np.ndarray:
        t = torch.empty(a.shape, dtype={2: torch.int16, 4: torch.float32}[a.dtype.itemsize]).pin_memory()
        out = t.numpy().view(a.dtype)
        out[...] = a
        pinned.keep.append(t)
        return out
    pinned.keep = []

    def measure(name, steps, warmup, full):
        """Times one workload.  full=False: device-resident leg only."""
        ctx = hb.Context(local_rank)
        ctx.set_stream(stream.cuda_stream)
        wl = WORKLOADS[name]()
        sharded = getattr(wl, "collective", False)        # the step has a real exchange between ranks
        strong = getattr(wl, "scaling", "weak") == "strong"
        if sharded:
            wl.setup(ctx, rank, pinned, world, dist)
        else:
            wl.setup(ctx, rank, pinned)

        def barrier():
            ctx.sync()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
                torch.cuda.synchronize()

        def timed(fn, n):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record(stream)
            for _ in range(n):
                fn(ctx)
            e1.record(stream)
            barrier()
            ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return float(ms.item())

        for _ in range(warmup):
            wl.step(ctx)
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        l0 = ctx.launches
        total_ms = timed(wl.step, steps)
        launches = ctx.launches - l0
        clocks = sampler.stop() if rank == 0 else None
        ms_per_step = total_ms / steps
        kern_ms = ms_per_step
        if sharded:
            value = wl.value(kern_ms, world)
            # per-GPU share of the algorithmic work (strong scaling splits it, weak repeats it)
            achieved = wl.flop / (world if strong else 1) / (kern_ms * 1e-3) / 1e12
        else:
            value = wl.flop * world / (kern_ms * 1e-3) / 1e12
            achieved = wl.flop / (kern_ms * 1e-3) / 1e12
        # Which measured peak applies: the burst figure for a short timed region, the sustained
        # (power-capped) one for a region of a second or more.  Both fractions are reported.
        long_run = total_ms > 1000.0
        if wl.bound == "tensor":
            peak = pk["bf16_sustained"] if long_run else pk["bf16_burst"]
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "peak_kind": ("sustained" if long_run else "burst") + " cuBLAS bf16, of " + pk["source"],
                    "frac_of_burst_peak": achieved / pk["bf16_burst"],
                    "frac_of_sustained_peak": achieved / pk["bf16_sustained"]}
        else:
            achieved = wl.bytes / (kern_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
                    "frac": achieved / pk["hbm"], "peak_kind": "STREAM-style copy, of " + pk["source"]}
        roof["traffic"] = NCU_TRAFFIC_BYTES.get(wl.name)
        roof["kernel"] = wl.kernel
        roof["kernel_ms"] = kern_ms
        if sharded:
            roof["note"] = "whole-step figure: algorithmic flop of the block / (n_gpus x step time), all kernels and collectives included"
        if hasattr(wl, "comm"):
            roof["collective"] = wl.comm
        res = {"metric": wl.metric, "value": value, "unit": wl.unit, "ms_per_step": ms_per_step, "steps": steps,
               "scaling": getattr(wl, "scaling", "weak"), "workload": wl.desc, "l2": wl.flush_note, "roofline": roof,
               "gpu_launches": launches, "clocks": clocks}
        if full:
            e2e_steps = max(3, min(steps, 10))
            wl.step_e2e(ctx)
            e2e_ms = timed(wl.step_e2e, e2e_steps) / e2e_steps
            e2e_value = wl.value(e2e_ms, world) if sharded else wl.flop * world / (e2e_ms * 1e-3) / 1e12
            res["e2e"] = {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": wl.h2d,
                          "d2h_bytes_per_step": wl.d2h, "ms_per_step": e2e_ms}
            if world == 1 and rank == 0 and not args.no_cpu_baseline:
                import oracle
                oracle.use_all_cores()
                v, sample = wl.cpu_sample()
                res["cpu_baseline"] = {"value": v, "unit": wl.unit, "cores": oracle.num_threads(), "kind": "port",
                                       "sample": sample}
        barrier()
        ctx.close()
        pinned.keep.clear()
        return res

    main_res = measure(args.workload, args.steps, args.warmup, True)
    extras = {}
    for name in [e for e in args.extras.split(",") if e and e != args.workload]:
        r = measure(name, max(3, min(args.steps, 20)), 3, False)
        extras[name] = {k: r[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "scaling", "roofline",
                                          "gpu_launches")}
    if rank == 0:
        line = {"metric": main_res["metric"], "value": main_res["value"], "unit": main_res["unit"], "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_res["ms_per_step"],
                "higher_is_better": True, "scaling": main_res["scaling"], "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic",
                "config": {"workload": main_res["workload"],
                           "parallelism": ("tp%d" % world if main_res["scaling"] == "strong" else
                                           ("dp%d" % world if args.workload == "mlp" else
                                            ("replicas only" if world > 1 else "single GPU"))),
                           "l2": main_res["l2"], "seed": SEED},
                "roofline": main_res["roofline"], "e2e": main_res["e2e"], "gpu_launches": main_res["gpu_launches"],
                "clocks": main_res["clocks"], "extras": extras}
        if "cpu_baseline" in main_res:
            line["cpu_baseline"] = main_res["cpu_baseline"]
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
