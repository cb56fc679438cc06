"""Reverse-mode differentiation over the model-IR nodes the training configuration uses
(matmul against a weight, GELU, MSE), and a data-parallel Adam trainer on top of it.

A :class:`Tape` records the forward nodes as they are launched; :meth:`Tape.backward`
replays them in reverse and launches the gradient kernels.  Every tensor stays on the
device; weights are kept as fp32 masters with fp32 Adam moments and a bf16 compute copy,
gradients are bf16 (also on the wire when data-parallel ranks sum them).

Weight layout: ``W`` is ``[out_features, in_features]`` row-major, i.e. the column-major
B operand of ``y = x @ W^T``.  The backward products reuse the same buffers through
strided views: ``dX = dY @ W`` reads W as an N-contiguous B operand and
``dW = dY^T @ X`` reads dY as an M-contiguous A operand, so no transposition pass runs.
"""
from __future__ import annotations

import os
from typing import List, Optional

import numpy as np

from . import _capi
from .model_ir import Context, Tensor


class Tape:
    def __init__(self, ctx: Context):
        self.ctx = ctx
        self.ops = []

    # -- forward nodes ------------------------------------------------------------
    def linear(self, x: Tensor, w_bf16: Tensor, out: Tensor, grad_w: Tensor, need_dx: bool = True) -> Tensor:
        """out[B, out] = x[B, in] @ W^T with W [out, in]."""
        self.ctx.matmul(x, w_bf16.T, out=out)
        self.ops.append(("linear", x, w_bf16, out, grad_w, need_dx))
        return out

    def gelu(self, z: Tensor, out: Tensor) -> Tensor:
        self.ctx.gelu(z, out=out)
        self.ops.append(("gelu", z, out))
        return out

    def mse(self, y: Tensor, target: Tensor, dy: Tensor, loss: Tensor):
        self.ctx.mse(y, target, dy=dy, loss=loss)
        self.ops.append(("mse", y, dy))
        return loss

    # -- backward -------------------------------------------------------------------
    def backward(self, scratch: List[Tensor], on_grad=None, on_layer_done=None):
        """Launches the gradient kernels.  `scratch` holds two [B, width] bf16 buffers used
        alternately for activation gradients.  `on_grad(grad_w)` is called right after each
        weight gradient is enqueued (the data-parallel trainer sums it there);
        `on_layer_done(grad_w)` once both products of a linear layer are enqueued, i.e. when
        nothing queued later reads that layer's weights (the trainer updates them there)."""
        ctx = self.ctx
        grads = {}                      # id(tensor) -> gradient tensor
        k = 0
        for op in reversed(self.ops):
            if op[0] == "mse":
                _, y, dy = op
                grads[id(y)] = dy
            elif op[0] == "gelu":
                _, z, out = op
                dout = grads[id(out)]
                dz = scratch[k % 2]
                k += 1
                ctx.gelu_backward(z, dout, out=ctx.wrap(dz.ptr, z.shape))
                grads[id(z)] = ctx.wrap(dz.ptr, z.shape)
            else:
                _, x, w, out, grad_w, need_dx = op
                dout = grads[id(out)]
                # dW[out, in] = dY^T[out, B] @ X[B, in]
                ctx.matmul(dout.T, x, out=grad_w)
                if on_grad:
                    on_grad(grad_w)
                if need_dx:
                    dx = scratch[k % 2]
                    k += 1
                    # dX[B, in] = dY[B, out] @ W[out, in]
                    ctx.matmul(dout, w, out=ctx.wrap(dx.ptr, x.shape))
                    grads[id(x)] = ctx.wrap(dx.ptr, x.shape)
                if on_layer_done:
                    on_layer_done(grad_w)
        self.ops.clear()


class MlpTrainer:
    """n-layer MLP (no biases, GELU between layers, none after the last), MSE loss, Adam."""

    def __init__(self, ctx: Context, width: int, batch: int, n_layers: int, weights_f32: List[np.ndarray],
                 world: int = 1, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, grads_base_ptr: Optional[int] = None,
                 algo: int = _capi.HB_AR_AUTO):
        self.ctx, self.width, self.batch, self.n, self.world = ctx, width, batch, n_layers, world
        self.lr, self.b1, self.b2, self.eps, self.algo = lr, beta1, beta2, eps, algo
        self.step_no = 0
        self.overlap_update = os.environ.get("HB_MLP_OVERLAP_UPDATE", "1") != "0"   # Adam under the backward products
        from .model_ir import f32_to_bf16_bits as to_bf16_bits
        self.w32 = [ctx.upload(np.ascontiguousarray(w, np.float32)) for w in weights_f32]
        self.wb = [ctx.upload(to_bf16_bits(w)) for w in weights_f32]
        zeros = np.zeros((width, width), np.float32)
        self.m = [ctx.upload(zeros) for _ in range(n_layers)]
        self.v = [ctx.upload(zeros) for _ in range(n_layers)]
        gbytes = width * width * 2
        if grads_base_ptr is None:
            self.grads = [ctx.empty((width, width)) for _ in range(n_layers)]
        else:   # gradients live in the peer-mapped buffer so the allreduce runs in place
            self.grads = [ctx.wrap(grads_base_ptr + i * gbytes, (width, width)) for i in range(n_layers)]
        self.z = [ctx.empty((batch, width)) for _ in range(n_layers)]
        self.h = [ctx.empty((batch, width)) for _ in range(n_layers - 1)]
        self.scratch = [ctx.empty((batch, width)) for _ in range(2)]
        self.dy = ctx.empty((batch, width))
        self.loss = ctx.empty((1,), _capi.HB_F32)

    @staticmethod
    def grad_bytes(width: int, n_layers: int) -> int:
        return n_layers * width * width * 2

    def step(self, x: Tensor, y: Tensor):
        """One forward + backward + (allreduce) + Adam step; everything is enqueued."""
        ctx = self.ctx
        tape = Tape(ctx)
        h = x
        for i in range(self.n):
            tape.linear(h, self.wb[i], self.z[i], self.grads[i], need_dx=i > 0)
            if i < self.n - 1:
                h = tape.gelu(self.z[i], self.h[i])
        tape.mse(self.z[-1], y, self.dy, self.loss)
        # each weight gradient is summed across ranks on the side stream while the main stream
        # goes on with the remaining backward products
        on_grad = (lambda g: ctx.all_reduce_async(g, self.algo)) if self.world > 1 else None
        self.step_no += 1
        layer_of = {id(g): i for i, g in enumerate(self.grads)}

        # The optimizer step of a layer is bound by HBM, the backward products by the tensor cores:
        # as soon as both products of a layer are enqueued (nothing later reads its weights), its
        # update goes to the side stream -- behind that layer's gradient sum, which is on the same
        # stream -- and runs under the products of the layers still to come.
        def update(grad_w):
            i = layer_of[id(grad_w)]
            ctx.adam_step(self.w32[i], self.m[i], self.v[i], self.grads[i], self.wb[i], self.step_no, self.lr, self.b1,
                          self.b2, self.eps, 1.0 / self.world, on_side_stream=self.overlap_update)
        tape.backward(self.scratch, on_grad, update)
        if self.world > 1 or self.overlap_update:
            ctx.side_join()
        return self.loss

    # -- checkpoint / resume ----------------------------------------------------------
    _MAGIC = "# habu_b200 mlp checkpoint v1"

    def save(self, path: str):
        """Writes the training state: one text header line per field, a blank line, then the
        raw little-endian fp32 tensors in order -- for each layer the master weights, the first
        and the second Adam moment.  The bf16 compute copies are not stored: they are the
        masters rounded to nearest even, and :meth:`load` rebuilds them."""
        ctx = self.ctx
        ctx.sync()
        with open(path, "wb") as f:
            head = [self._MAGIC, f"width {self.width}", f"layers {self.n}", f"step {self.step_no}",
                    f"lr {self.lr!r}", f"beta1 {self.b1!r}", f"beta2 {self.b2!r}", f"eps {self.eps!r}",
                    "dtype f32le", "order w,m,v per layer", ""]
            f.write(("\n".join(head) + "\n").encode())
            for i in range(self.n):
                for t in (self.w32[i], self.m[i], self.v[i]):
                    f.write(np.ascontiguousarray(ctx.download(t), "<f4").tobytes())

    def load(self, path: str):
        """Restores a state written by :meth:`save` into this trainer (same width and depth);
        the next :meth:`step` then equals, bit for bit, the step the saving trainer would have
        taken.  Raises ValueError on a foreign, truncated or mismatching file."""
        from .model_ir import f32_to_bf16_bits
        ctx = self.ctx
        with open(path, "rb") as f:
            blob = f.read()
        cut = blob.find(b"\n\n")
        if cut < 0 or not blob.startswith(self._MAGIC.encode()):
            raise ValueError(f"{path}: not a habu_b200 mlp checkpoint")
        fields = dict(line.split(" ", 1) for line in blob[:cut].decode().splitlines()[1:])
        if int(fields["width"]) != self.width or int(fields["layers"]) != self.n:
            raise ValueError(f"{path}: checkpoint is {fields['layers']} x {fields['width']}, trainer is {self.n} x {self.width}")
        body = memoryview(blob)[cut + 2:]
        per = self.width * self.width * 4
        if len(body) != 3 * self.n * per:
            raise ValueError(f"{path}: truncated ({len(body)} tensor bytes, expected {3 * self.n * per})")
        import ctypes as C
        from .model_ir import _lib
        k = 0
        for i in range(self.n):
            for t in (self.w32[i], self.m[i], self.v[i]):
                a = np.frombuffer(body[k * per:(k + 1) * per], "<f4").astype(np.float32)
                k += 1
                ctx._check(_lib.hb_upload(ctx._h, C.c_void_p(t.ptr), a.ctypes.data_as(C.c_void_p), a.nbytes))
                ctx.sync()
                if t is self.w32[i]:
                    wb = f32_to_bf16_bits(a)
                    ctx._check(_lib.hb_upload(ctx._h, C.c_void_p(self.wb[i].ptr), wb.ctypes.data_as(C.c_void_p), wb.nbytes))
                    ctx.sync()
        self.step_no = int(fields["step"])
        self.lr, self.b1, self.b2, self.eps = (float(fields[k]) for k in ("lr", "beta1", "beta2", "eps"))
