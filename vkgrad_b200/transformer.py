"""Decoder-only transformer on the B200 kernels.

Same classes and constructor arguments as the reference's transformer.py --
`TCtx` (transformer.py:23), `LayerNorm` (44), `Dense` (74), `Attention` (107),
`Block` (189), `GPT(ctx, B, T, D, H, n_layer, vocab, pad_vocab, tie)` (253) with
`params()`, `forward`, `record(ids, targets, graph, backward, seg, weights)` and
`read_loss()` -- and the same layout conventions (residual stream (B*T, D) fp32,
GEMM operands fp16, fp32 accumulation, vocabulary padded to a multiple of 16 and
masked in the loss).

The op plan is fused where the reference's is not:
  * every Dense is one GEMM whose epilogue adds the bias and, as needed, keeps
    the pre-activation, applies GELU, adds the residual and narrows to fp16
    (replacing bias_gelu / residual / to16 / bias_gelu_bwd16 dispatches);
  * q, k, v are addressed in place inside the (rows, 3D) projection through
    batch strides, and the attention output / gradients are written straight
    into the merged layout, so split_qkv, merge_heads, split_heads and
    merge_qkv_grad disappear (transformer.py:141-186);
  * layernorm backward adds the residual-branch gradient, emits the fp16 copy
    and reduces dgamma/dbeta in the same pass (replacing add + to16 + two
    column sums, transformer.py:63-71, 230-242);
  * score / dP / dS scratch is shared by all layers; only P is kept per layer.
A static loss scale can be applied in the loss kernel (`loss_scale`); parameter
gradients then carry that factor until AdamW divides it out.
"""

import zlib

import numpy as np

from ._lib import ACT_GELU, ACT_NONE, F16, F32, TUNE_SM_LIMIT
from .autograd import Ctx, Param
from .kernels import gemm, gemm_group
from .tkernels import make_transformer_kernels
from .vk import _check

NCHUNK = 32  # kept for callers that pass it to col_sum_chunk (transformer.py:20)
CAUSAL_BLOCK = 128  # row-tile height of the GEMM: where its causal K ranges stop
GROUP_DW = True        # GPT.record issues the dW GEMMs of all blocks as one grouped launch
FUSED_HEAD_DIM = 64  # head size the fused attention kernels are written for
_LN_FUSED_MAX_D = 1536  # shared-memory limit of the fused dgamma/dbeta reduction


class TCtx(Ctx):
    """Ctx plus the transformer kernel dictionary and per-model shared scratch."""

    def __init__(self, dev, tune=False, scalar_only=None):
        super().__init__(dev, tune, scalar_only)
        self.TK = make_transformer_kernels(dev)
        self._shared = {}

    def shared_buf(self, tag, nbytes):
        """A buffer every layer may reuse for values that die within the layer."""
        b = self._shared.get(tag)
        if b is None or b.size < nbytes:
            b = self.buf(nbytes)
            self._shared[tag] = b
        return b


class LayerNorm:
    def __init__(self, ctx, rows, D, name=""):
        self.ctx, self.rows, self.D = ctx, rows, D
        self.g = Param(ctx, (D,), np.ones(D, np.float32), name + ".g", no_decay=True)
        self.b = Param(ctx, (D,), np.zeros(D, np.float32), name + ".b", no_decay=True)
        self.y16 = ctx.buf(rows * D * 2)
        self.mu = ctx.buf(rows * 4)
        self.rstd = ctx.buf(rows * 4)
        self.dx = ctx.buf(rows * D * 4)
        self.dx16 = ctx.buf(rows * D * 2)
        self._scratch = None

    def forward(self, x32, graph=None):
        self.x32 = x32
        lib, h = self.ctx.dev.lib, self.ctx.dev.handle

        def go():
            _check(lib.vkg_layernorm(h, x32.dptr, self.g.w32.dptr, self.b.w32.dptr, self.y16.dptr,
                                     self.mu.dptr, self.rstd.dptr, self.rows, self.D), "layernorm")
        self.ctx.launch(graph, go, "layernorm", self.rows * self.D * 6)
        return self.y16

    def can_sum_dx(self):
        """Whether backward() can also produce the column sums of dx (the bias gradient
        of the Dense that consumes dx) in the same pass."""
        return self.D % 128 == 0 and self.D <= 1024

    def backward(self, dy32, graph=None, dres=None, dxsum=None):
        """dx = LN'(dy) (+ dres); also writes dx16, g.g32 and b.g32, and, when dxsum is
        given (see can_sum_dx), the column sums of dx into it.  Returns dx."""
        c, dev = self.ctx, self.ctx.dev
        lib, h = dev.lib, dev.handle
        R, D = self.rows, self.D
        x32 = self.x32
        dres_p = None if dres is None else dres.dptr
        if dxsum is not None and not self.can_sum_dx():
            raise ValueError("dxsum needs D to be a multiple of 128 and at most 1024")
        dxsum_p = None if dxsum is None else dxsum.dptr
        if D <= _LN_FUSED_MAX_D:
            # partial parameter sums; private to this layer because the final pass may be a
            # deferred one (GPT.record collects them into one launch)
            if self._scratch is None:
                self._scratch = c.buf(lib.vkg_layernorm_bwd_scratch_floats(R, D) * 4)
            scratch = self._scratch

            def go():
                _check(lib.vkg_layernorm_bwd(h, dy32.dptr, x32.dptr, self.g.w32.dptr, self.mu.dptr,
                                             self.rstd.dptr, dres_p, self.dx.dptr, self.dx16.dptr,
                                             None, None, self.g.g32.dptr, self.b.g32.dptr, dxsum_p,
                                             scratch.dptr, R, D), "layernorm_bwd")
            c.launch(graph, go, "layernorm_bwd", R * D * 18)
        else:
            dyxh = c.shared_buf("ln_dyxh", R * D * 2)
            dy16 = c.shared_buf("ln_dy16", R * D * 2)

            def go():
                _check(lib.vkg_layernorm_bwd(h, dy32.dptr, x32.dptr, self.g.w32.dptr, self.mu.dptr,
                                             self.rstd.dptr, dres_p, self.dx.dptr, self.dx16.dptr,
                                             dyxh.dptr, dy16.dptr, None, None, None, None, R, D),
                       "layernorm_bwd")
            c.launch(graph, go, "layernorm_bwd", R * D * 22)
            c.col_sum(dyxh, self.g.g32, D, R, graph=graph)
            c.col_sum(dy16, self.b.g32, D, R, graph=graph)
        return self.dx


class Dense:
    """y = x @ W + b with fp16 in; the caller chooses what the epilogue does with
    the output (transformer.py:74-104)."""

    def __init__(self, ctx, rows, in_f, out_f, name="", scale=None):
        self.ctx, self.rows, self.in_f, self.out_f = ctx, rows, in_f, out_f
        self.name = name
        # seeded by the layer's name through a stable hash: the same weights in every process
        # (the reference draws from hash(name), which Python salts per process,
        # autograd.py:172-173 / transformer.py:80-82; its tests overwrite the weights anyway)
        rng = np.random.default_rng(zlib.crc32(name.encode()))
        s = scale if scale is not None else np.sqrt(2.0 / in_f)
        w = (rng.standard_normal((in_f, out_f)) * s).astype(np.float32)
        self.W = Param(ctx, (in_f, out_f), w, name + ".W")
        self.b = Param(ctx, (out_f,), np.zeros(out_f, np.float32), name + ".b", no_decay=True)
        self.acc = None
        self.dx32 = None
        self._colsum_scratch = None

    def forward(self, x16, graph=None, out=None, c_dtype=F32, act=ACT_NONE, pre=None,
                residual=None, c2=None):
        """out = epilogue(x16 @ W + b).  Without `out`, an fp32 buffer is used
        (bias already added), like the reference's acc followed by its bias add."""
        self.x16 = x16
        if out is None:
            if self.acc is None:
                self.acc = self.ctx.buf(self.rows * self.out_f * 4)
            out = self.acc
        gemm(self.ctx.dev, x16, self.W.w16, out, self.rows, self.out_f, self.in_f, graph=graph,
             c_dtype=c_dtype, bias=self.b.w32, act=act, pre=pre, residual=residual, c2=c2,
             name=f"{self.name}.fwd")
        return out

    def backward(self, dy16, need_dx=True, graph=None, dx=None, dx_dtype=F32, dact_z=None,
                 dact=ACT_NONE, bias_grad_done=False, dx_colsum=None, dw_sink=None):
        """bias_grad_done: the producer of dy16 already wrote b.g32 (LayerNorm.backward's
        dxsum, or a GEMM's dx_colsum), so the column-sum pass is skipped.
        dx_colsum: fp32 buffer that receives the column sums of dx as stored -- the bias
        gradient of the layer below when dx is that layer's dY.
        dw_sink: a list; the dW GEMM is appended to it instead of being launched, for one
        grouped launch over all layers (the caller keeps x16 and dy16 intact until then)."""
        c, dev = self.ctx, self.ctx.dev
        R, I, O = self.rows, self.in_f, self.out_f
        if dw_sink is not None:
            dw_sink.append((self.x16, dy16, self.W.g32, I, O, R, dict(trans_a=True)))
        else:
            gemm(dev, self.x16, dy16, self.W.g32, I, O, R, trans_a=True, graph=graph,
                 name=f"{self.name}.dW")
        if need_dx:
            if dx is None:
                if self.dx32 is None:
                    self.dx32 = c.buf(R * I * 4)
                dx, dx_dtype = self.dx32, F32
            cs = None
            if dx_colsum is not None:
                # private, because the final pass over it may be a deferred one
                if self._colsum_scratch is None:
                    self._colsum_scratch = c.buf(dev.lib.vkg_gemm_colsum_scratch_floats(R, I) * 4)
                cs = self._colsum_scratch
            gemm(dev, dy16, self.W.w16, dx, R, I, O, trans_b=True, graph=graph, c_dtype=dx_dtype,
                 dact_z=dact_z, dact=dact, colsum=dx_colsum, colsum_scratch=cs, name=f"{self.name}.dX")
        if not bias_grad_done:
            c.col_sum(dy16, self.b.g32, O, R, graph=graph)
        return dx if need_dx else None


class Attention:
    """Causal multi-head attention as batched GEMMs over (batch, head) plus the
    row softmax (transformer.py:107-186), with heads addressed by strides."""

    def __init__(self, ctx, B, T, D, H, name="", fused=None):
        self.ctx, self.B, self.T, self.D, self.H = ctx, B, T, D, H
        self.hd = D // H
        self.rows = B * T
        self.nbh = B * H
        self.scale = 1.0 / np.sqrt(self.hd)
        self.name = name
        # head dimension 64 (GPT-2 shapes) runs the fused tcgen05 attention kernels:
        # no T x T tensor is ever written.  Other head sizes use batched GEMMs + softmax.
        self.fused = (self.hd == FUSED_HEAD_DIM) if fused is None else bool(fused)
        self.qkv = Dense(ctx, self.rows, D, 3 * D, name + ".qkv")
        self.proj = Dense(ctx, self.rows, D, D, name + ".proj", scale=np.sqrt(2.0 / D) * 0.5)
        att = self.nbh * T * T
        self.qkv16 = ctx.buf(self.rows * 3 * D * 2)
        self.ao16 = ctx.buf(self.rows * D * 2)
        self.dao16 = ctx.buf(self.rows * D * 2)
        self.dqkv16 = ctx.buf(self.rows * 3 * D * 2)
        self._dbias_scratch = None
        if self.fused:
            self.lse2 = ctx.buf(self.nbh * T * 4)
            self.delta = ctx.shared_buf("attn_delta", self.nbh * T * 4)
            return
        self.p16 = ctx.buf(att * 2)
        # dead after the layer's softmax / softmax backward: shared by all layers
        self.scores = ctx.shared_buf("attn_scores", att * 4)
        self.dp32 = ctx.shared_buf("attn_dp", att * 4)
        self.ds16 = ctx.shared_buf("attn_ds", att * 2)

    def _bgemm(self, a, b, c, m, n, k, graph, ta=False, tb=False, a_in_qkv=None, b_in_qkv=None,
               c_in_qkv=None, a_merged=False, b_merged=False, c_merged=False, c_dtype=F32,
               causal=0, name="attn"):
        """One GEMM per (head, batch): nb0 = H heads, nb1 = B sequences.

        *_in_qkv = i selects slice i (0 q, 1 k, 2 v) of a (rows, 3D) matrix;
        *_merged addresses a (rows, D) matrix by head; otherwise the operand is a
        dense (B*H, T, T) stack."""
        T, D, H, hd = self.T, self.D, self.H, self.hd

        def addr(in_qkv, merged, ld_dense):
            if in_qkv is not None:
                return dict(off=in_qkv * D, ld=3 * D, s=(hd, T * 3 * D))
            if merged:
                return dict(off=0, ld=D, s=(hd, T * D))
            return dict(off=0, ld=ld_dense, s=(T * T, H * T * T))
        A = addr(a_in_qkv, a_merged, T)
        Bm = addr(b_in_qkv, b_merged, T)
        Cm = addr(c_in_qkv, c_merged, T)
        return gemm(self.ctx.dev, a, b, c, m, n, k, ta, tb, graph=graph, nb0=H, nb1=self.B,
                    lda=A["ld"], ldb=Bm["ld"], ldc=Cm["ld"], sa=A["s"], sb=Bm["s"], sc=Cm["s"],
                    a_off=A["off"], b_off=Bm["off"], c_off=Cm["off"], c_dtype=c_dtype,
                    causal=causal, name=f"{self.name}.{name}")

    def forward(self, x16, graph=None, seg=None, out=None, residual=None):
        """Returns proj(attn(x)) + bias (+ residual) in fp32 (`out` or proj.acc)."""
        c, lib, h = self.ctx, self.ctx.dev.lib, self.ctx.dev.handle
        T, hd = self.T, self.hd
        self.qkv.forward(x16, graph=graph, out=self.qkv16, c_dtype=F16)
        self._seg = seg
        if self.fused:
            seg_f = None if seg is None else seg.dptr

            def fwd():
                _check(lib.vkg_attn_fwd(h, self.qkv16.dptr, seg_f, self.ao16.dptr, self.lse2.dptr,
                                        self.B, T, self.H, hd, float(self.scale)), "attn_fwd")
            c.launch(graph, fwd, "attn_fwd", self.rows * self.D * 8)
            return self.proj.forward(self.ao16, graph=graph, out=out, residual=residual)
        # scores = Q K^T per head; tiles wholly above the diagonal are never computed,
        # and nothing downstream reads past the 128-wide block that holds the diagonal
        self._bgemm(self.qkv16, self.qkv16, self.scores, T, T, hd, graph, tb=True,
                    a_in_qkv=0, b_in_qkv=1, causal=1, name="qk")
        seg_p = None if seg is None else seg.dptr

        def soft():
            _check(lib.vkg_attn_softmax(h, self.scores.dptr, seg_p, self.p16.dptr, self.nbh * T, T,
                                        self.H, float(self.scale), CAUSAL_BLOCK), "attn_softmax")
        c.launch(graph, soft, "attn_softmax", self.nbh * T * T * 6)
        # out = P V, written head-merged as fp16
        self._bgemm(self.p16, self.qkv16, self.ao16, T, hd, T, graph, b_in_qkv=2, c_merged=True,
                    c_dtype=F16, causal=2, name="pv")
        return self.proj.forward(self.ao16, graph=graph, out=out, residual=residual)

    def backward(self, dy16, graph=None, proj_bias_grad_done=False, dw_sink=None):
        """dy16: gradient of the projection's output.  Returns d(ln1 output), fp32."""
        c, lib, h = self.ctx, self.ctx.dev.lib, self.ctx.dev.handle
        T, hd = self.T, self.hd
        self.proj.backward(dy16, need_dx=True, graph=graph, dx=self.dao16, dx_dtype=F16,
                           bias_grad_done=proj_bias_grad_done, dw_sink=dw_sink)
        if self.fused:
            seg_f = None if self._seg is None else self._seg.dptr

            # the kernels that write dqkv also fold its column sums: the qkv bias gradient
            if self._dbias_scratch is None:    # private: its final pass may be a deferred one
                self._dbias_scratch = c.buf(4 * lib.vkg_attn_bwd_dbias_scratch_floats(
                    self.B, T, self.H, hd))
            scratch = self._dbias_scratch

            def bwd():
                _check(lib.vkg_attn_bwd(h, self.qkv16.dptr, self.dao16.dptr, self.ao16.dptr,
                                        self.lse2.dptr, seg_f, self.dqkv16.dptr, self.delta.dptr,
                                        self.qkv.b.g32.dptr, scratch.dptr,
                                        self.B, T, self.H, hd, float(self.scale)), "attn_bwd")
            c.launch(graph, bwd, "attn_bwd", self.rows * self.D * 16)
            return self.qkv.backward(self.dqkv16, need_dx=True, graph=graph, bias_grad_done=True,
                                     dw_sink=dw_sink)
        # dV = P^T dO  -> slice 2 of dqkv
        self._bgemm(self.p16, self.dao16, self.dqkv16, T, hd, T, graph, ta=True, b_merged=True,
                    c_in_qkv=2, c_dtype=F16, causal=3, name="dv")
        # dP = dO V^T
        self._bgemm(self.dao16, self.qkv16, self.dp32, T, T, hd, graph, tb=True, a_merged=True,
                    b_in_qkv=2, causal=1, name="dp")

        def soft_bwd():
            _check(lib.vkg_attn_softmax_bwd(h, self.dp32.dptr, self.p16.dptr, self.ds16.dptr,
                                            self.nbh * T, T, float(self.scale), CAUSAL_BLOCK),
                   "attn_softmax_bwd")
        c.launch(graph, soft_bwd, "attn_softmax_bwd", self.nbh * T * T * 8)
        # dQ = dS K -> slice 0 ; dK = dS^T Q -> slice 1
        self._bgemm(self.ds16, self.qkv16, self.dqkv16, T, hd, T, graph, b_in_qkv=1, c_in_qkv=0,
                    c_dtype=F16, causal=2, name="dq")
        self._bgemm(self.ds16, self.qkv16, self.dqkv16, T, hd, T, graph, ta=True, b_in_qkv=0,
                    c_in_qkv=1, c_dtype=F16, causal=3, name="dk")
        return self.qkv.backward(self.dqkv16, need_dx=True, graph=graph, dw_sink=dw_sink)


class Block:
    """Pre-LN block: x + attn(ln1(x)), then + fc2(gelu(fc1(ln2(.)))) (transformer.py:189-250)."""

    def __init__(self, ctx, B, T, D, H, name="", fused_attention=None):
        self.ctx = ctx
        self.rows = B * T
        self.D = D
        self.ln1 = LayerNorm(ctx, self.rows, D, name + ".ln1")
        self.attn = Attention(ctx, B, T, D, H, name + ".attn", fused=fused_attention)
        self.ln2 = LayerNorm(ctx, self.rows, D, name + ".ln2")
        self.fc1 = Dense(ctx, self.rows, D, 4 * D, name + ".fc1")
        self.fc2 = Dense(ctx, self.rows, 4 * D, D, name + ".fc2",
                         scale=np.sqrt(2.0 / (4 * D)) * 0.5)
        self.res1 = ctx.buf(self.rows * D * 4)
        self.res2 = ctx.buf(self.rows * D * 4)
        self.z1 = ctx.buf(self.rows * 4 * D * 4)
        self.h16 = ctx.buf(self.rows * 4 * D * 2)
        # fc1's dY: kept per block, the grouped dW launch at the end of the backward reads it
        self.dh16 = ctx.buf(self.rows * 4 * D * 2)

    def forward(self, x32, graph=None, seg=None):
        self.x32 = x32
        h = self.ln1.forward(x32, graph=graph)
        self.attn.forward(h, graph=graph, seg=seg, out=self.res1, residual=x32)
        h2 = self.ln2.forward(self.res1, graph=graph)
        self.fc1.forward(h2, graph=graph, out=self.h16, c_dtype=F16, act=ACT_GELU, pre=self.z1)
        self.fc2.forward(self.h16, graph=graph, out=self.res2, residual=self.res1)
        return self.res2

    def backward(self, d32, d16, graph=None, fc2_bias_grad_done=False, below=None, dw_sink=None):
        """d32/d16: gradient of the block output in both precisions.
        Returns the gradient of the block input as (fp32, fp16).

        fc2_bias_grad_done: whoever produced d16 already reduced its column sums into
        fc2.b.g32.  below: the block that consumes this block's input gradient; its fc2
        bias gradient is then produced by this block's last layernorm backward."""
        # MLP branch; the residual sends the same gradient down both paths.
        # fc2's dX is fc1's dY: its column sums are fc1's bias gradient, taken in the epilogue
        self.fc2.backward(d16, graph=graph, dx=self.dh16, dx_dtype=F16, dact_z=self.z1,
                          dact=ACT_GELU, bias_grad_done=fc2_bias_grad_done,
                          dx_colsum=self.fc1.b.g32, dw_sink=dw_sink)
        dln2 = self.fc1.backward(self.dh16, graph=graph, bias_grad_done=True, dw_sink=dw_sink)
        fuse = self.ln2.can_sum_dx()
        dres1 = self.ln2.backward(dln2, graph=graph, dres=d32,
                                  dxsum=self.attn.proj.b.g32 if fuse else None)
        # attention branch
        dln1 = self.attn.backward(self.ln2.dx16, graph=graph, proj_bias_grad_done=fuse,
                                  dw_sink=dw_sink)
        dx = self.ln1.backward(dln1, graph=graph, dres=dres1,
                               dxsum=below.fc2.b.g32 if (below is not None and fuse) else None)
        return dx, self.ln1.dx16

    def params(self):
        for p in (self.ln1.g, self.ln1.b, self.ln2.g, self.ln2.b,
                  self.attn.qkv.W, self.attn.qkv.b, self.attn.proj.W, self.attn.proj.b,
                  self.fc1.W, self.fc1.b, self.fc2.W, self.fc2.b):
            yield p


class GPT:
    def __init__(self, ctx, B, T, D, H, n_layer, vocab, pad_vocab=None, tie=False,
                 loss_scale=1.0, fused_attention=None):
        self.ctx, self.B, self.T, self.D = ctx, B, T, D
        self.rows = B * T
        self.vocab = vocab
        self.pad_vocab = pad_vocab or ((vocab + 15) // 16) * 16
        self.loss_scale = float(loss_scale)
        rng = np.random.default_rng(1234)
        self.tok = Param(ctx, (self.pad_vocab, D),
                         (rng.standard_normal((self.pad_vocab, D)) * 0.02).astype(np.float32), "tok")
        self.pos = Param(ctx, (T, D), (rng.standard_normal((T, D)) * 0.02).astype(np.float32), "pos")
        self.x0 = ctx.buf(self.rows * D * 4)
        self.blocks = [Block(ctx, B, T, D, H, f"b{i}", fused_attention=fused_attention)
                       for i in range(n_layer)]
        self.lnf = LayerNorm(ctx, self.rows, D, "lnf")
        self.tie = tie
        self.logits = ctx.buf(self.rows * self.pad_vocab * 4)
        if tie:
            self.dh32 = ctx.buf(self.rows * D * 4)
        else:
            self.head = Dense(ctx, self.rows, D, self.pad_vocab, "head", scale=0.02)
        self.dlog16 = ctx.buf(self.rows * self.pad_vocab * 2)
        self.loss = ctx.buf(self.rows * 4, "cached")

    def params(self):
        yield self.tok
        yield self.pos
        for b in self.blocks:
            yield from b.params()
        yield self.lnf.g
        yield self.lnf.b
        if not self.tie:
            yield self.head.W
            yield self.head.b

    def n_params(self):
        return sum(p.n for p in self.params())

    def n_stages(self):
        return 2 * len(self.blocks) + 3

    def forward(self, ids_buf, graph=None, seg=None):
        """Logits (rows, pad_vocab) fp32.  seg: optional (B*T,) u32, the index in its
        row where each token's packed sample starts.  graph: a Graph, None for
        eager, or a stage -> Graph callable (see record)."""
        c, lib, h = self.ctx, self.ctx.dev.lib, self.ctx.dev.handle
        g = graph if callable(graph) else (lambda stage: graph)
        seg_p = None if seg is None else seg.dptr

        def emb():
            _check(lib.vkg_embed(h, self.tok.w32.dptr, self.pos.w32.dptr, ids_buf.dptr, seg_p,
                                 self.x0.dptr, self.rows * self.D, self.D, self.T), "embed")
        c.launch(g(0), emb, "embed", self.rows * self.D * 12)
        x = self.x0
        for i, b in enumerate(self.blocks):
            x = b.forward(x, graph=g(i), seg=seg)
        L = len(self.blocks)
        hf = self.lnf.forward(x, graph=g(L))
        self.h16 = hf
        R, V, D = self.rows, self.pad_vocab, self.D
        if self.tie:
            # logits = h tok^T; tok is stored V x D, hence trans_b
            gemm(c.dev, hf, self.tok.w16, self.logits, R, V, D, trans_b=True, graph=g(L),
                 name="head.fwd")
        else:
            self.head.forward(hf, graph=g(L), out=self.logits)
        return self.logits

    def record(self, ids_buf, targets_buf, graph, backward=True, seg=None, weights=None,
               flush_after=(), sm_limit_after_flush=0):
        """Record the loss and, unless backward=False, every gradient.

        graph may be a stage -> Graph callable that spreads the step over several
        submits, with the reference's stage numbering (transformer.py:339-345):
        i < L embedding (stage 0) and block i forward; L head and loss; L+1 head and
        lnf backward; L+2+k block L-1-k backward; 2L+2 embedding backward.
        Stage graphs must be finished in stage order: the backward collects its short final
        passes from stage L+1 on and runs them in stage 2L+2 (vkg_finals_defer / _flush act
        when a graph is finished, not when it is recorded).
        weights: optional per-row loss weights replacing the 1/rows mean; the loss
        buffer then holds each row's unweighted cross entropy, 0 where the weight
        is 0 (kernels.py:793-827).
        flush_after: block indices; once the backward of such a block is recorded, the dW GEMMs
        collected so far are issued as a group and the pending final passes run, in that
        block's stage graph -- every gradient of the blocks above it (and of lnf) is then
        complete, so a data-parallel step can start summing that part of the bucket while the
        blocks below are still in their backward.  sm_limit_after_flush > 0 caps the persistent
        kernels recorded after the first flush at that many CTAs (room for the collective).
        """
        c, lib, h = self.ctx, self.ctx.dev.lib, self.ctx.dev.handle
        g = graph if callable(graph) else (lambda stage: graph)
        L = len(self.blocks)
        R, V, D = self.rows, self.pad_vocab, self.D
        logits = self.forward(ids_buf, graph=g, seg=seg)
        w_p = None if weights is None else weights.dptr
        # per-row weights carry their own normalisation; the static loss scale multiplies both
        scale = self.loss_scale / R if weights is None else self.loss_scale

        def ce():
            _check(lib.vkg_softmax_ce(h, logits.dptr, targets_buf.dptr, w_p, self.dlog16.dptr, None,
                                      self.loss.dptr, R, V, self.vocab, scale), "softmax_ce")
        c.launch(g(L), ce, "softmax_ce", R * V * 10)
        if not backward:
            return
        gh = g(L + 1)
        # the short second passes of the bias and layernorm-parameter sums (49 in a 12-layer
        # model) are collected and run as one launch after the last kernel of the backward
        c.launch(gh, lambda: _check(lib.vkg_finals_defer(h, 1), "finals_defer"), "finals_defer")
        if self.tie:
            # dh = dlogits tok ; head's share of dtok = dlogits^T h (overwrites tok.g32)
            gemm(c.dev, self.dlog16, self.tok.w16, self.dh32, R, D, V, graph=gh, name="head.dX")
            gemm(c.dev, self.dlog16, self.h16, self.tok.g32, V, D, R, trans_a=True, graph=gh,
                 name="head.dW")
            d = self.dh32
        else:
            d = self.head.backward(self.dlog16, need_dx=True, graph=gh)

            def zero_tok():
                _check(lib.vkg_memset0(h, self.tok.g32.dptr, self.tok.n * 4), "zero tok grad")
            c.launch(gh, zero_tok, "zero", self.tok.n * 4)
        fuse = self.lnf.can_sum_dx() and L > 0
        d32 = self.lnf.backward(d, graph=gh, dxsum=self.blocks[-1].fc2.b.g32 if fuse else None)
        d16 = self.lnf.dx16
        # the blocks' dW GEMMs (4 per block, 18..72 tiles each) are collected and issued as
        # one grouped launch once every dY exists
        dw_sink = [] if GROUP_DW and L > 0 else None
        flush_after = set(int(i) for i in flush_after)
        limited = False
        for k in range(L):
            i = L - 1 - k
            gk = g(L + 2 + k)
            d32, d16 = self.blocks[i].backward(d32, d16, graph=gk, fc2_bias_grad_done=fuse,
                                               below=self.blocks[i - 1] if i > 0 else None,
                                               dw_sink=dw_sink)
            if i in flush_after and i > 0:
                if dw_sink:
                    gemm_group(c.dev, dw_sink, graph=gk, name=f"blocks{i}+.dW")
                    dw_sink = []
                c.launch(gk, lambda: _check(lib.vkg_finals_flush(h), "finals_flush"), "finals_flush")
                c.launch(gk, lambda: _check(lib.vkg_finals_defer(h, 1), "finals_defer"),
                         "finals_defer")
                if sm_limit_after_flush > 0 and not limited:
                    limited = True
                    c.launch(gk, lambda: _check(lib.vkg_set_tuning(h, TUNE_SM_LIMIT,
                                                                   int(sm_limit_after_flush)),
                                                "sm_limit"), "sm_limit")
        ge = g(2 * L + 2)
        if dw_sink:
            gemm_group(c.dev, dw_sink, graph=ge, name="blocks.dW")
        seg_p = None if seg is None else seg.dptr

        # rows that share a token (or a position) are added in row order by one warp, so the
        # whole step is bit-reproducible; table widths the kernel has no instance for keep
        # the reference's atomic scatter-add
        det = D % 128 == 0 and D <= 1024
        if det and getattr(self, "_emb_scratch", None) is None:
            self._emb_scratch = c.buf(lib.vkg_embed_bwd_scratch_bytes(R))

        def emb_bwd():
            _check(lib.vkg_memset0(h, self.pos.g32.dptr, self.pos.n * 4), "zero pos grad")
            if det:
                _check(lib.vkg_embed_bwd_det(h, d32.dptr, ids_buf.dptr, seg_p, self.tok.g32.dptr,
                                             self.pos.g32.dptr, self._emb_scratch.dptr, R * D, D,
                                             self.T), "embed_bwd_det")
                return
            _check(lib.vkg_embed_bwd(h, d32.dptr, ids_buf.dptr, seg_p, self.tok.g32.dptr,
                                     self.pos.g32.dptr, R * D, D, self.T), "embed_bwd")
        c.launch(ge, emb_bwd, "embed_bwd", R * D * 12)
        c.launch(ge, lambda: _check(lib.vkg_finals_flush(h), "finals_flush"), "finals_flush",
                 4 * sum(p.n for p in self.params() if len(p.shape) == 1))
        if limited:
            c.launch(ge, lambda: _check(lib.vkg_set_tuning(h, TUNE_SM_LIMIT, 0), "sm_limit"),
                     "sm_limit")

    def read_loss(self):
        self.loss.invalidate()
        return float(self.loss.array(np.float32, (self.rows,)).mean())
