"""Layers, optimiser and the recorded training step for the MLP path.

Same public classes as the reference's autograd.py -- `Ctx` (autograd.py:44),
`Param` (111), `Linear` (159), `MLP` (231), `AdamW` (304), `TrainStep` (346) --
with the same constructor arguments, buffers (`w32`/`w16`/`g32`/`m`/`v`) and
methods, so the reference's examples and tests drive it unchanged.

What differs is where the work happens.  The reference runs matmul, then a
bias+GELU kernel, then (backward) a GELU' kernel, a column sum and two matmuls,
each a separate dispatch with a DRAM round trip between them.  Here a Linear
forward is ONE tcgen05 GEMM whose epilogue adds the bias, keeps the fp32
pre-activation, applies the activation and narrows to fp16; the backward's dX
GEMM multiplies by the activation derivative of the layer below in its
epilogue and writes fp16 directly; AdamW is one multi-tensor launch for all
parameters instead of one dispatch per tensor (autograd.py:331-335).
"""

import ctypes as C

import zlib

import numpy as np

from . import _lib
from ._lib import ACT_GELU, ACT_NONE, ACT_RELU, F16, F32
from .kernels import CONFIGS, TILE, Matmul, gemm, make_kernels
from .vk import VkError, _check

_ACTS = {"gelu": ACT_GELU, "relu": ACT_RELU, None: ACT_NONE, "none": ACT_NONE}


def pick_config(m, n, k, trans_a=False, trans_b=False, min_groups=12):
    """Reference-shaped (sg, wm, wn, lds) for a shape (autograd.py:22-41).

    The tcgen05 kernel picks its own 128 x {64..256} tile per call, so this only
    reports the widest reference tile that divides the shape; it raises VkError
    when none does, as the reference does.
    """
    best = None
    for sg, wm, wn, lds in CONFIGS:
        if lds:
            continue
        bm, bn = sg * wm * TILE, wn * TILE
        if m % bm or n % bn or k % TILE:
            continue
        score = ((m // bm) * (n // bn) >= min_groups, bm * bn)
        if best is None or score > best[0]:
            best = (score, (sg, wm, wn, False))
    if best is None:
        raise VkError(f"no matmul tile fits {m}x{n}x{k}")
    return best[1]


class Ctx:
    """Owns the device, the kernel dictionary, a matmul cache and its buffers."""

    def __init__(self, dev, tune=False, scalar_only=None):
        self.dev = dev
        self.K = make_kernels(dev)
        self.tune = tune
        self.scalar_only = False   # every B200 has tensor cores; there is no scalar path
        self._mm = {}
        self._owned = []

    def matmul(self, m, n, k, trans_a=False, trans_b=False, batched=False, nbatch=1):
        key = (m, n, k, trans_a, trans_b, batched, nbatch)
        if key not in self._mm:
            if self.tune:
                from .kernels import autotune_matmul
                mm, _ = autotune_matmul(self.dev, m, n, k, trans_a, trans_b,
                                        batched=batched, nbatch=nbatch)
            else:
                mm = Matmul(self.dev, trans_a=trans_a, trans_b=trans_b, batched=batched, tile_n=0)
            self._mm[key] = mm
        return self._mm[key]

    def buf(self, nbytes, kind="device"):
        b = self.dev.buffer(nbytes, kind)
        self._owned.append(b)
        return b

    def zeros(self, n_floats):
        b = self.buf(n_floats * 4, "device")
        _check(self.dev.lib.vkg_memset0(self.dev.handle, b.dptr, n_floats * 4), "zeros")
        return b

    def launch(self, graph, thunk, name, nbytes=0):
        """Record `thunk` into `graph`, or run it now and return GPU seconds."""
        if graph is not None:
            graph.add(thunk, name, nbytes)
            return 0.0
        return self.dev.run_op(thunk)

    def col_sum(self, src, dst, ncol, nrow, graph=None, f16=True, accumulate=False):
        """dst[c] = sum over rows of src[r, c]; deterministic two-stage reduction.

        Replaces col_sum_zero + col_sum_chunk(16) (transformer.py:30-36)."""
        lib, h = self.dev.lib, self.dev.handle
        scratch = self.dev.scratch(lib.vkg_col_sum_scratch_floats(ncol, nrow) * 4)
        dt = F16 if f16 else F32

        def go():
            _check(lib.vkg_col_sum_det(h, src.dptr, dt, dst.dptr, scratch.dptr, ncol, nrow,
                                       1 if accumulate else 0), "col_sum")
        return self.launch(graph, go, "col_sum", nrow * ncol * (2 if f16 else 4))

    def destroy(self):
        self.dev.sync()
        # a recording abandoned half way must not leave deferred passes behind
        self.dev.lib.vkg_finals_defer(self.dev.handle, -1)
        for b in self._owned:
            b.destroy()
        self._owned = []
        self._mm.clear()


class Param:
    """fp32 master, fp16 mirror for the GEMMs, fp32 gradient, Adam moments
    (autograd.py:111-156).  The mirror is refreshed inside the optimiser step."""

    def __init__(self, ctx, shape, init=None, name="", no_decay=False):
        self.ctx = ctx
        self.shape = tuple(shape)
        self.n = int(np.prod(shape))
        self.name = name
        self.no_decay = no_decay
        self.w32 = ctx.buf(self.n * 4, "cached")
        self.w16 = ctx.buf(self.n * 2, "device")
        self.g32 = ctx.buf(self.n * 4, "device")
        self.m = ctx.zeros(self.n)
        self.v = ctx.zeros(self.n)
        w = self.w32.array(np.float32, self.shape)
        w[...] = 0 if init is None else init
        self.w32.flush()
        self.sync16()

    def sync16(self):
        d = self.ctx.dev
        _check(d.lib.vkg_cast16(d.handle, self.w32.dptr, self.w16.dptr, self.n), "cast16")
        d.sync()

    def numpy(self):
        self.w32.invalidate()
        return self.w32.array(np.float32, self.shape)

    def set(self, arr):
        self.w32.array(np.float32, self.shape)[...] = arr
        self.w32.flush()
        self.sync16()

    def grad_numpy(self):
        """Copy of the gradient, for checking."""
        d = self.ctx.dev
        out = np.empty(self.shape, np.float32)
        tmp = d.buffer(self.n * 4, "cached")
        try:
            d.copy(self.g32, tmp, self.n * 4)
            tmp.invalidate()
            out[...] = tmp.array(np.float32, self.shape)
        finally:
            tmp.destroy()
        return out


class Linear:
    """y = act(x @ W + b), or the same without the activation (autograd.py:159-228).

    forward is one GEMM (bias, saved pre-activation, activation and the fp16
    narrowing in the epilogue).  backward_pre takes the gradient of the
    pre-activation: dW GEMM into W.g32, column sum into b.g32, and the dX GEMM,
    which folds the activation derivative of the layer below into its epilogue
    when that layer is given.
    """

    def __init__(self, ctx, batch, in_f, out_f, activation=True, need_dx=True, name="",
                 act="gelu"):
        self.ctx, self.name = ctx, name
        self.batch, self.in_f, self.out_f = batch, in_f, out_f
        self.activation = activation
        self.act = _ACTS[act] if activation else ACT_NONE
        self.need_dx = need_dx
        # seeded by the layer's name through a stable hash: the same weights in every process
        # (the reference draws from hash(name), which Python salts per process,
        # autograd.py:172-173 / transformer.py:80-82; its tests overwrite the weights anyway)
        rng = np.random.default_rng(zlib.crc32(name.encode()))
        w = (rng.standard_normal((in_f, out_f)) * np.sqrt(2.0 / in_f)).astype(np.float32)
        self.W = Param(ctx, (in_f, out_f), w, name + ".W")
        self.b = Param(ctx, (out_f,), np.zeros(out_f, np.float32), name + ".b", no_decay=True)
        self.z = ctx.buf(batch * out_f * 4)       # pre-activation, kept for backward
        self.y16 = ctx.buf(batch * out_f * 2)     # activation, feeds the next GEMM
        self.dz16 = ctx.buf(batch * out_f * 2)
        self.dz32 = ctx.buf(batch * out_f * 4)
        self.dx32 = ctx.buf(batch * in_f * 4) if need_dx else None
        self.dx16 = ctx.buf(batch * in_f * 2) if need_dx else None
        self.x16 = None

    def forward(self, x16, tape=None, graph=None):
        self.x16 = x16
        B, I, O = self.batch, self.in_f, self.out_f
        mm = self.ctx.matmul(B, O, I)
        x_dev = _stage(mm, x16, B * I * 2, graph)
        if self.activation:
            gemm(self.ctx.dev, x_dev, self.W.w16, self.y16, B, O, I, graph=graph, c_dtype=F16,
                 bias=self.b.w32, pre=self.z, act=self.act, name=f"{self.name}.fwd")
            out = self.y16
        else:
            gemm(self.ctx.dev, x_dev, self.W.w16, self.z, B, O, I, graph=graph, c_dtype=F32,
                 bias=self.b.w32, name=f"{self.name}.fwd")
            out = self.z
        self._x_dev = x_dev
        if tape is not None:
            tape.append(self.backward)
        return out

    def backward(self, dout16, dout32, graph=None):
        """Reference semantics: dout is dLoss/dOutput in both precisions.
        Returns (None, dx32)."""
        if self.activation:
            lib, h = self.ctx.dev.lib, self.ctx.dev.handle
            n = self.batch * self.out_f

            def go():
                _check(lib.vkg_bias_act_bwd(h, dout32.dptr, self.z.dptr, self.dz16.dptr,
                                            self.dz32.dptr, n, self.act), "act_bwd")
            self.ctx.launch(graph, go, "bias_act_bwd", n * 14)
            g16, g32 = self.dz16, self.dz32
        else:
            g16, g32 = dout16, dout32
        self.backward_pre(g16, g32, graph=graph)
        return None, self.dx32

    def backward_pre(self, g16, g32=None, graph=None, below=None):
        """g16 (and optionally g32) is dLoss/d(pre-activation).  Returns what the
        layer below consumes: its pre-activation gradient in fp16 when `below`
        is that layer (derivative fused), else this layer's dx32."""
        c, dev = self.ctx, self.ctx.dev
        B, I, O = self.batch, self.in_f, self.out_f
        # dW = X^T dZ: X is stored batch x in_f, i.e. K x M -> trans_a.
        gemm(dev, self._x_dev, g16, self.W.g32, I, O, B, trans_a=True, graph=graph,
             name=f"{self.name}.dW")
        if g32 is not None:
            c.col_sum(g32, self.b.g32, O, B, graph=graph, f16=False)
        else:
            c.col_sum(g16, self.b.g32, O, B, graph=graph, f16=True)
        if not self.need_dx:
            return None
        # dX = dZ W^T: W is stored in_f x out_f, i.e. N x K -> trans_b.
        if below is not None and below.activation:
            gemm(dev, g16, self.W.w16, self.dx16, B, I, O, trans_b=True, graph=graph,
                 c_dtype=F16, dact_z=below.z, dact=below.act, name=f"{self.name}.dX")
            return self.dx16
        gemm(dev, g16, self.W.w16, self.dx32, B, I, O, trans_b=True, graph=graph,
             name=f"{self.name}.dX")
        return self.dx32


def _stage(mm, x, nbytes, graph):
    """Copy a host-mapped GEMM operand into HBM (TMA reads device memory only)."""
    if getattr(x, "kind", "device") not in ("shared", "bar"):
        return x
    dev = mm.dev
    tmp = dev.staging(("in", x.dptr), nbytes)

    def go():
        _check(dev.lib.vkg_copy(dev.handle, tmp.dptr, x.dptr, nbytes), "stage input")
    if graph is not None:
        graph.add(go, "stage_input", nbytes)
        graph.n_dispatch -= 1
    else:
        go()
    return tmp


class MLP:
    """Hidden layers with an activation, a linear head feeding softmax + CE
    (autograd.py:231-301).  n_classes is padded to pad_classes; padded logits are
    masked in the loss kernel.  act is "gelu" (the reference's) or "relu"."""

    def __init__(self, ctx, batch, sizes, n_classes, pad_classes=16, act="gelu"):
        assert pad_classes >= n_classes and pad_classes % 8 == 0
        self.ctx, self.batch = ctx, batch
        self.n_classes, self.pad = n_classes, pad_classes
        self.layers = []
        for i in range(len(sizes) - 1):
            self.layers.append(Linear(ctx, batch, sizes[i], sizes[i + 1], activation=True,
                                      need_dx=(i > 0), name=f"fc{i}", act=act))
        self.layers.append(Linear(ctx, batch, sizes[-1], pad_classes, activation=False,
                                  need_dx=True, name="head"))
        self.dlog16 = ctx.buf(batch * pad_classes * 2)
        self.dlog32 = ctx.buf(batch * pad_classes * 4)
        self.loss = ctx.buf(batch * 4, "cached")

    def params(self):
        for l in self.layers:
            yield l.W
            yield l.b

    def logits(self, x16, tape=None, graph=None):
        h = x16
        for l in self.layers:
            h = l.forward(h, None, graph=graph)
        return h

    def _loss(self, logits, labels_buf, graph):
        lib, hnd = self.ctx.dev.lib, self.ctx.dev.handle
        B, pad, ncls = self.batch, self.pad, self.n_classes

        def go():
            _check(lib.vkg_softmax_ce(hnd, logits.dptr, labels_buf.dptr, None, self.dlog16.dptr,
                                      self.dlog32.dptr, self.loss.dptr, B, pad, ncls, 1.0 / B),
                   "softmax_ce")
        self.ctx.launch(graph, go, "softmax_ce", B * pad * 10)

    def _backward(self, graph):
        g16, g32 = self.dlog16, self.dlog32
        for i in reversed(range(len(self.layers))):
            below = self.layers[i - 1] if i > 0 else None
            g16 = self.layers[i].backward_pre(g16, g32, graph=graph, below=below)
            g32 = None

    def record(self, x16, labels_buf, graph):
        """Record forward, loss and backward; read the loss with read_loss()."""
        logits = self.logits(x16, graph=graph)
        self._loss(logits, labels_buf, graph)
        self._backward(graph)

    def read_loss(self):
        self.loss.invalidate()
        return float(self.loss.array(np.float32, (self.batch,)).mean())

    def forward_backward(self, x16, labels_buf):
        """Eager: every kernel launched and waited for on its own."""
        logits = self.logits(x16)
        self._loss(logits, labels_buf, None)
        loss = self.read_loss()
        self._backward(None)
        return loss

    def predict(self, x16):
        logits = self.logits(x16)
        d = self.ctx.dev
        tmp = d.buffer(self.batch * self.pad * 4, "cached")
        try:
            d.copy(logits, tmp, self.batch * self.pad * 4)
            tmp.invalidate()
            out = tmp.array(np.float32, (self.batch, self.pad))[:, :self.n_classes]
            return out.argmax(1).copy()
        finally:
            tmp.destroy()


class AdamW:
    """Fused AdamW over every parameter in one launch (reference: one dispatch per
    tensor, autograd.py:304-343).  Step-varying scalars live in a mapped buffer
    the kernel reads, so a recorded step stays valid as they change
    (autograd.py:313-323).  hp[6] is an extra gradient scale (0 = none): the
    1/(workers * loss_scale) the data-parallel path folds in."""

    def __init__(self, ctx, params, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.01):
        self.ctx, self.params = ctx, list(params)
        self.lr, self.b1, self.b2, self.eps, self.wd = lr, b1, b2, eps, wd
        self.t = 0
        self.grad_scale = 0.0
        self.hp = ctx.buf(8 * 4, "shared")
        self.hpv = self.hp.array(np.float32)
        self._tables = {}
        self._set_hp(lr)

    def _set_hp(self, lr):
        bc1 = 1 - self.b1 ** max(self.t, 1)
        bc2 = 1 - self.b2 ** max(self.t, 1)
        self.hpv[:7] = [lr, self.b1, self.b2, bc1, bc2, self.eps, self.grad_scale]
        self.hp.flush()

    def advance(self, lr=None):
        self.t += 1
        self._set_hp(self.lr if lr is None else lr)

    def _get_table(self, params):
        key = tuple((p.w32.dptr, p.g32.dptr, p.m.dptr, p.v.dptr, p.w16.dptr) for p in params)
        if key in self._tables:
            return self._tables[key]
        d = self.ctx.dev
        n = len(params)
        arr = lambda vals: (C.c_void_p * n)(*vals)
        sizes = (C.c_int64 * n)(*[p.n for p in params])
        wds = (C.c_float * n)(*[0.0 if p.no_decay else self.wd for p in params])
        t = C.c_void_p()
        _check(d.lib.vkg_adamw_table_create(
            d.handle, n, arr([k[0] for k in key]), arr([k[1] for k in key]),
            arr([k[2] for k in key]), arr([k[3] for k in key]), arr([k[4] for k in key]),
            sizes, wds, C.byref(t)), "adamw_table")
        self._tables[key] = t      # tables of older pointer sets stay alive for their graphs
        return t

    def record(self, graph, params=None):
        """params: update only these (a subset of the optimiser's parameters, e.g. one part of
        a gradient bucket whose all-reduce has finished); default all."""
        self._launch(graph, params)

    def _launch(self, graph, params=None):
        d = self.ctx.dev
        params = self.params if params is None else list(params)
        table = self._get_table(params)

        def go():
            _check(d.lib.vkg_adamw_multi(d.handle, table, self.hp.dptr), "adamw")
        self.ctx.launch(graph, go, "adamw_multi", 30 * sum(p.n for p in params))

    def step(self, lr=None):
        """Eager step."""
        self.advance(lr)
        self._launch(None)


class TrainStep:
    """Forward, backward and optimiser recorded once and replayed (autograd.py:346-366).
    Per-step data is whatever the caller writes into xbuf/ybuf (mapped memory)
    and the optimiser's hyper-parameter buffer."""

    def __init__(self, model, opt, xbuf, ybuf):
        self.model, self.opt = model, opt
        self.graph = model.ctx.dev.graph("train_step")
        model.record(xbuf, ybuf, self.graph)
        opt.record(self.graph)
        self.graph.finish()
        self.n_dispatch = self.graph.n_dispatch

    def __call__(self, lr=None):
        self.opt.advance(lr)
        dt = self.graph.submit()
        return self.model.read_loss(), dt
