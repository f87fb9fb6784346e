"""Kernel objects with the call conventions of the reference's kernels.py.

`Matmul` keeps the constructor and `__call__(a, b, c, m, n, k, repeat, graph,
nbatch, strides)` of kernels.py:232-315; `make_kernels(dev)` returns the same
dictionary of fused elementwise ops as kernels.py:699-862, each called as
`K[name](buffers, n, *push, repeat=1, graph=None)` like Elementwise.__call__
(kernels.py:687-693).  Behind them there is no shader generator: every call
goes through ctypes into the ahead-of-time compiled sm_100a library, and the
matmul is one persistent tcgen05 kernel whose tile shape is picked per call.

`gemm()` is the wider entry the fused training step uses: batch strides in two
levels and the fused epilogue (bias, activation, activation derivative,
residual, f16 copy) of vkg_gemm.
"""

import ctypes as C
import json
import os

import numpy as np

from . import _lib
from ._lib import ACT_GELU, ACT_NONE, ACT_RELU, BF16, F16, F32, GemmArgs
from .vk import VkError, _check

TILE = 16  # granularity the reference's shapes come in (kernels.py:18)

# (sg, wm, wn, lds) tuples of the reference (kernels.py:326-331).  They name
# RDNA3 workgroup shapes; here they only select the N-tile hint via wn.
CONFIGS = [(sg, wm, wn, lds)
           for sg in (1, 2, 4, 8)
           for wm in (1, 2, 3, 4)
           for wn in (1, 2, 3, 4, 6, 8)
           for lds in (False, True)
           if sg * 32 <= 1024 and wm * wn <= 16]

TILE_N_CHOICES = (64, 128, 192, 256)
SPLIT_K_MAX_TILE_BYTES = 32 << 20   # outputs larger than this already fill the GPU


def _ptr(buf):
    if buf is None:
        return None
    if isinstance(buf, int):
        return buf
    if buf.dptr is None:
        raise VkError("buffer was destroyed")
    return buf.dptr


def _gemm_args(dev, a, b, c, m, n, k, trans_a=False, trans_b=False,
               nb0=1, nb1=1, lda=None, ldb=None, ldc=None, sa=(0, 0), sb=(0, 0), sc=(0, 0),
               a_off=0, b_off=0, c_off=0, in_dtype=F16, c_dtype=F32, bias=None, act=ACT_NONE,
               pre=None, dact_z=None, dact=ACT_NONE, residual=None, c2=None, tile_n=0,
               max_ctas=0, alpha=1.0, split_k=0, causal=0, cta_pair=0, colsum=None,
               colsum_scratch=None):
    """Fill a vkg_gemm_args (include/vkgrad_b200.h).  Offsets are in elements and apply to
    C, c2, pre, dact_z and residual alike."""
    args = GemmArgs()
    args.trans_a, args.trans_b = int(bool(trans_a)), int(bool(trans_b))
    args.M, args.N, args.K = int(m), int(n), int(k)
    args.nb0, args.nb1 = int(nb0), int(nb1)
    args.in_dtype = in_dtype
    esz_c = 4 if c_dtype == F32 else 2
    args.A = _ptr(a) + 2 * int(a_off)
    args.lda = int(lda if lda is not None else (m if trans_a else k))
    args.sA0, args.sA1 = int(sa[0]), int(sa[1])
    args.B = _ptr(b) + 2 * int(b_off)
    args.ldb = int(ldb if ldb is not None else (k if trans_b else n))
    args.sB0, args.sB1 = int(sb[0]), int(sb[1])
    args.C = _ptr(c) + esz_c * int(c_off)
    args.ldc = int(ldc if ldc is not None else n)
    args.sC0, args.sC1 = int(sc[0]), int(sc[1])
    args.c_dtype = c_dtype
    args.act = act
    args.C2 = None if c2 is None else _ptr(c2) + 2 * int(c_off)
    args.bias = _ptr(bias)
    args.pre = None if pre is None else _ptr(pre) + 4 * int(c_off)
    args.dact_z = None if dact_z is None else _ptr(dact_z) + 4 * int(c_off)
    args.dact = dact
    args.residual = None if residual is None else _ptr(residual) + 4 * int(c_off)
    args.tile_n = int(tile_n)
    args.max_ctas = int(max_ctas)
    args.alpha = float(alpha)
    args.split_k = int(split_k)
    args.causal = int(causal)
    args.cta_pair = int(cta_pair)
    if colsum is not None:
        # column sums of the stored output, folded by the epilogue warps; the partial rows
        # live in scratch until the final pass has read them: the launch's own, or, under
        # vkg_finals_defer, the collected one, which needs scratch no other call touches
        args.colsum = _ptr(colsum)
        need = dev.lib.vkg_gemm_colsum_scratch_floats(int(m), int(n)) * 4
        if colsum_scratch is not None and colsum_scratch.size < need:
            raise VkError(f"colsum_scratch holds {colsum_scratch.size} bytes, {need} needed")
        args.colsum_scratch = (dev.scratch(need) if colsum_scratch is None else colsum_scratch).dptr
        args.split_k = 1
        split_k = 1
    plain = (bias is None and pre is None and dact_z is None and residual is None and c2 is None
             and act == ACT_NONE and c_dtype == F32 and alpha == 1.0)
    if split_k != 1 and plain and nb0 * nb1 == 1 and m * n * 4 <= SPLIT_K_MAX_TILE_BYTES:
        # few output tiles, long K (the dW shapes): give the library room to split K
        ws = dev.scratch((int(split_k) if split_k > 1 else 8) * m * n * 4)
        args.workspace = ws.dptr
        args.workspace_bytes = ws.size
    return args


def gemm(dev, a, b, c, m, n, k, trans_a=False, trans_b=False, graph=None, repeat=1, name="gemm",
         **kw):
    """C = op(A) op(B) with the fused epilogue of vkg_gemm (include/vkgrad_b200.h).

    Keyword arguments as in _gemm_args: a head's slice of a wider matrix can be
    addressed in place through the element offsets.  Returns GPU seconds when run
    eagerly, 0.0 when recorded.
    """
    args = _gemm_args(dev, a, b, c, m, n, k, trans_a=trans_a, trans_b=trans_b, **kw)
    lib, h = dev.lib, dev.handle

    def go():
        _check(lib.vkg_gemm(h, C.byref(args)), f"{name} {m}x{n}x{k}")

    if graph is not None:
        nb = args.nb0 * args.nb1
        esz_c = 4 if args.c_dtype == F32 else 2
        graph.add(go, name, nb * (2 * m * k + 2 * k * n + esz_c * m * n))
        graph.mm_split.append((nb * 2 * (m * k + k * n), nb * m * n * esz_c))
        return 0.0
    return dev.run_op(go, repeat)


def gemm_group(dev, problems, graph=None, repeat=1, name="gemm_group", cta_pair=1):
    """Many independent plain GEMMs in one launch (vkg_gemm_group_*): `problems` is a list of
    (a, b, c, m, n, k, kwargs) as for gemm(), fp32 outputs without epilogue extras.  Used for
    the dW of every Linear of a model (autograd.py:217-219): few tiles each, thousands
    together.  The launch table is built here, once; the returned thunk only launches."""
    n = len(problems)
    arr = (GemmArgs * n)()
    keep = []
    for i, pr in enumerate(problems):
        args = _gemm_args(dev, *pr[:6], **dict(pr[6], split_k=1))
        keep.append(args)
        C.memmove(C.byref(arr, i * C.sizeof(GemmArgs)), C.byref(args), C.sizeof(GemmArgs))
    lib, h = dev.lib, dev.handle
    table = dev.buffer(lib.vkg_gemm_group_table_bytes(n), "device")
    units = C.c_int32(0)
    _check(lib.vkg_gemm_group_prepare(h, arr, n, table.dptr, int(cta_pair), C.byref(units)),
           f"{name} prepare")

    def go():
        _check(lib.vkg_gemm_group_launch(h, table.dptr, n, units.value), name)

    go.table = table       # lives as long as the recorded launch
    if graph is not None:
        total = 0
        for args in keep:
            m, nn, k = args.M, args.N, args.K
            total += 2 * m * k + 2 * k * nn + 4 * m * nn
            graph.mm_split.append((2 * (m * k + k * nn), 4 * m * nn))
        graph.add(go, name, total)
        return 0.0
    return dev.run_op(go, repeat)


class Matmul:
    """One matmul configuration (kernels.py:232-315).

    sg/wm/wn are accepted for compatibility; bm/bn report the reference's
    workgroup tile so callers that print them keep working, but the kernel
    always computes 128 x tile_n tiles and accepts ragged edges.  wn selects the
    N tile when it maps onto one (wn*16 in {64,128,192,256}); otherwise the
    library chooses from the shape.
    """

    def __init__(self, dev, sg=4, wm=2, wn=2, trans_a=False, trans_b=False,
                 capture_stats=False, lds=False, bk=32, batched=False, acc16=False,
                 group_m=0, tile_n=None, in_dtype=F16):
        if lds and (trans_a or trans_b or batched):
            raise ValueError("LDS variant has no transposed or batched path")
        self.dev = dev
        self.sg, self.wm, self.wn = sg, wm, wn
        self.trans_a, self.trans_b = trans_a, trans_b
        self.lds, self.bk, self.batched = lds, bk, batched
        self.acc16, self.group_m = acc16, group_m
        self.bm, self.bn = sg * wm * TILE, wn * TILE
        self.in_dtype = in_dtype
        if tile_n is None:
            tile_n = self.bn if self.bn in TILE_N_CHOICES else 0
        self.tile_n = tile_n
        self.name = (f"mm_tcgen05_n{tile_n or 'auto'}"
                     f"{'_ta' if trans_a else ''}{'_tb' if trans_b else ''}"
                     f"{'_bat' if batched else ''}{'_a16' if acc16 else ''}")
        self.push_size = 24 if batched else 12
        self.kernel = self

    def fits(self, m, n, k):
        """Alignment the TMA descriptors need: 16-byte row pitches."""
        lda = m if self.trans_a else k
        ldb = k if self.trans_b else n
        return m > 0 and n > 0 and k > 0 and n % 8 == 0 and lda % 8 == 0 and ldb % 8 == 0

    def __call__(self, a, b, c, m, n, k, repeat=1, graph=None, nbatch=1, strides=(0, 0, 0)):
        if not self.fits(m, n, k):
            raise VkError(f"{self.name}: shape {m}x{n}x{k} needs n and the operand row "
                          f"lengths to be multiples of 8")
        nb = nbatch if self.batched else 1
        sa, sb_, sc = (strides if self.batched else (0, 0, 0))
        # Host-mapped ("shared") operands are staged into HBM first: the TMA
        # loads of the GEMM only ever see device memory.
        stage = []
        a_dev, b_dev = a, b
        if getattr(a, "kind", "device") in ("shared", "bar"):
            nbytes = (nb - 1) * sa * 2 + m * k * 2
            a_dev = self.dev.staging((id(self), "a", a.dptr), nbytes)
            stage.append((a_dev, a, nbytes))
        if getattr(b, "kind", "device") in ("shared", "bar"):
            nbytes = (nb - 1) * sb_ * 2 + n * k * 2
            b_dev = self.dev.staging((id(self), "b", b.dptr), nbytes)
            stage.append((b_dev, b, nbytes))
        lib, h = self.dev.lib, self.dev.handle
        c_dtype = F16 if self.acc16 else F32
        if stage:
            def copies():
                for dst, src, nbytes in stage:
                    _check(lib.vkg_copy(h, dst.dptr, src.dptr, nbytes), "stage operand")
            if graph is not None:
                graph.add(copies, "stage_operands", sum(s[2] for s in stage))
                graph.n_dispatch -= 1
            else:
                copies()
        return gemm(self.dev, a_dev, b_dev, c, m, n, k, self.trans_a, self.trans_b, graph=graph,
                    repeat=repeat, nb0=nb, sa=(sa, 0), sb=(sb_, 0), sc=(sc, 0),
                    in_dtype=self.in_dtype, c_dtype=c_dtype, tile_n=self.tile_n, name=self.name)

    def traffic_bytes(self, m, n, k, nbatch=1):
        """Compulsory traffic: each operand once, the output once."""
        nb = nbatch if self.batched else 1
        return nb * (2 * m * k + 2 * k * n + (2 if self.acc16 else 4) * m * n)

    def flops(self, m, n, k):
        return 2 * m * n * k

    def statistics(self):
        return {}

    def destroy(self):
        pass


_WARMED = set()


def warmup(dev, seconds=1.0, force=False):
    """Sustained load so clocks settle before timing (kernels.py:353-381)."""
    import time
    if not force and id(dev) in _WARMED:
        return 0.0
    m = n = k = 2048
    a = dev.buffer(m * k * 2, "device")
    b = dev.buffer(k * n * 2, "device")
    c = dev.buffer(m * n * 4, "device")
    mm = Matmul(dev)
    t0 = time.perf_counter()
    try:
        while time.perf_counter() - t0 < seconds:
            mm(a, b, c, m, n, k, repeat=20)
    finally:
        for x in (a, b, c):
            x.destroy()
    _WARMED.add(id(dev))
    return time.perf_counter() - t0


_TUNE_CACHE = os.path.join(os.path.dirname(os.path.abspath(__file__)), ".autotune.json")


def autotune_matmul(dev, m, n, k, trans_a=False, trans_b=False, reps=3, verbose=False,
                    use_cache=True, batched=False, nbatch=1):
    """Time the N-tile choices for one shape and return (Matmul, info).

    Same contract as kernels.py:450-603 (info carries config, tflops, ms,
    evaluated, pruned, tile), but the search space is the four tile widths of
    the tcgen05 kernel, timed round-robin over equal GPU time.
    """
    key = (f"{dev.name}|{m}x{n}x{k}|ta{int(trans_a)}tb{int(trans_b)}"
           f"{'|bat' + str(nbatch) if batched else ''}")
    cache = {}
    if use_cache and os.path.exists(_TUNE_CACHE):
        with open(_TUNE_CACHE) as f:
            cache = json.load(f)
    if key in cache:
        e = cache[key]
        return Matmul(dev, trans_a=trans_a, trans_b=trans_b, batched=batched,
                      tile_n=e["tile"][1]), e
    warmup(dev)
    nb = nbatch if batched else 1
    call = dict(nbatch=nb, strides=(m * k, k * n, m * n)) if batched else {}
    a = dev.buffer(nb * m * k * 2, "device")
    b = dev.buffer(nb * k * n * 2, "device")
    c = dev.buffer(nb * m * n * 4, "device")
    try:
        cands = [Matmul(dev, trans_a=trans_a, trans_b=trans_b, batched=batched, tile_n=t)
                 for t in TILE_N_CHOICES if t <= max(64, ((n + 63) // 64) * 64)]
        warm = {id(mm): mm(a, b, c, m, n, k, **call) for mm in cands}
        best_t = {id(mm): float("inf") for mm in cands}
        for _ in range(reps):
            for mm in cands:
                r = max(1, int(0.02 / max(warm[id(mm)], 1e-6)))
                best_t[id(mm)] = min(best_t[id(mm)], mm(a, b, c, m, n, k, repeat=r, **call) / r)
        results = []
        for mm in cands:
            t = best_t[id(mm)]
            tf = mm.flops(m, n, k) * nb / t / 1e12
            results.append({"config": [4, 2, mm.tile_n // 16], "lds": False, "tflops": tf,
                            "ms": t * 1e3, "tile": [128, mm.tile_n], "group_m": 0})
            if verbose:
                print(f"    tile 128x{mm.tile_n:3d}  {tf:8.2f} TFLOPS  {t * 1e6:8.1f} us")
        results.sort(key=lambda r: -r["tflops"])
        best = dict(results[0], evaluated=len(results), pruned=0)
        if use_cache:
            cache[key] = best
            tmp = _TUNE_CACHE + f".{os.getpid()}.tmp"
            with open(tmp, "w") as f:
                json.dump(cache, f, indent=2, sort_keys=True)
            os.replace(tmp, _TUNE_CACHE)
        return Matmul(dev, trans_a=trans_a, trans_b=trans_b, batched=batched,
                      tile_n=best["tile"][1]), best
    finally:
        for x in (a, b, c):
            x.destroy()


def matmul_reference(a, b, trans_a=False, trans_b=False):
    """What the kernel computes, in numpy: 16-bit inputs widened, fp32 product."""
    lhs = np.asarray(a, dtype=np.float32)
    rhs = np.asarray(b, dtype=np.float32)
    if trans_a:
        lhs = lhs.T
    if trans_b:
        rhs = rhs.T
    return np.matmul(lhs, rhs)


class Elementwise:
    """A named op with the reference's calling convention (kernels.py:668-696).

    `launch(buffers, n, *args)` enqueues the C entry point on the device stream.
    """

    def __init__(self, dev, name, launch, n_buffers, prepare=None):
        self.dev, self.name, self._launch, self.n_buffers = dev, name, launch, n_buffers
        # prepare(buffers, n, *args) runs when the op is called or recorded (never
        # inside a capture) and may allocate; its result is passed to launch.
        self._prepare = prepare
        self.kernel = self

    def __call__(self, buffers, n, *args, repeat=1, graph=None):
        if len(buffers) != self.n_buffers:
            raise VkError(f"{self.name}: expected {self.n_buffers} buffers, got {len(buffers)}")
        bufs = list(buffers)
        extra = () if self._prepare is None else (self._prepare(bufs, int(n), *args),)

        def go():
            self._launch(bufs, int(n), *args, *extra)

        if graph is not None:
            graph.add(go, self.name, sum(b.size for b in bufs))
            return 0.0
        return self.dev.run_op(go, repeat)

    def destroy(self):
        pass


def _op(dev, name, n_buffers, fn):
    return Elementwise(dev, name, fn, n_buffers)


def make_kernels(dev):
    """The MLP-step ops under the reference's names (kernels.py:699-862)."""
    lib, h = dev.lib, dev.handle
    K = {}

    def ck(status, what):
        _check(status, what)

    K["bias_gelu"] = _op(dev, "bias_gelu", 4, lambda b, n, ncol: ck(
        lib.vkg_bias_act(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, n, int(ncol), ACT_GELU),
        "bias_gelu"))
    K["bias_relu"] = _op(dev, "bias_relu", 4, lambda b, n, ncol: ck(
        lib.vkg_bias_act(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, n, int(ncol), ACT_RELU),
        "bias_relu"))
    K["bias_gelu_bwd"] = _op(dev, "bias_gelu_bwd", 4, lambda b, n: ck(
        lib.vkg_bias_act_bwd(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, n, ACT_GELU),
        "bias_gelu_bwd"))
    K["bias_gelu_bwd16"] = _op(dev, "bias_gelu_bwd16", 3, lambda b, n: ck(
        lib.vkg_bias_act_bwd(h, b[0].dptr, b[1].dptr, b[2].dptr, None, n, ACT_GELU),
        "bias_gelu_bwd16"))
    K["bias_relu_bwd"] = _op(dev, "bias_relu_bwd", 4, lambda b, n: ck(
        lib.vkg_bias_act_bwd(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, n, ACT_RELU),
        "bias_relu_bwd"))
    K["bias"] = _op(dev, "bias", 3, lambda b, n, ncol: ck(
        lib.vkg_bias(h, b[0].dptr, b[1].dptr, b[2].dptr, n, int(ncol)), "bias"))
    # col_sum: n is the column count, push is the row count (kernels.py:753-761)
    K["col_sum"] = _op(dev, "col_sum", 2, lambda b, n, nrow: ck(
        lib.vkg_col_sum(h, b[0].dptr, b[1].dptr, n, int(nrow)), "col_sum"))
    K["softmax_ce"] = _op(dev, "softmax_ce", 5, lambda b, n, stride, ncls: ck(
        lib.vkg_softmax_ce(h, b[0].dptr, b[1].dptr, None, b[2].dptr, b[3].dptr, b[4].dptr,
                           n, int(stride), int(ncls), 1.0 / n), "softmax_ce"))
    K["softmax_ce_w"] = _op(dev, "softmax_ce_w", 5, lambda b, n, stride, ncls: ck(
        lib.vkg_softmax_ce(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, None, b[4].dptr,
                           n, int(stride), int(ncls), 0.0), "softmax_ce_w"))
    K["adamw"] = _op(dev, "adamw", 6, lambda b, n, wd: ck(
        lib.vkg_adamw(h, b[0].dptr, b[1].dptr, b[2].dptr, b[3].dptr, b[4].dptr, b[5].dptr,
                      n, float(wd)), "adamw"))
    K["zero"] = _op(dev, "zero", 1, lambda b, n: ck(
        lib.vkg_memset0(h, b[0].dptr, n * 4), "zero"))
    K["cast16"] = _op(dev, "cast16", 2, lambda b, n: ck(
        lib.vkg_cast16(h, b[0].dptr, b[1].dptr, n), "cast16"))
    return K
