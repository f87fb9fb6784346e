"""GEMM trio parity on the GPU, through the C ABI: the reference's own kernel tests
(test_kernels.py) against the golden fixture and the CPU oracle, plus ragged,
batched and fused-epilogue cases the reference cannot express."""

import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402
from oracle import vkgrad_numpy as orc  # noqa: E402

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
TOL = 2e-3  # the reference's kernel tolerance: max|got-ref| / max|ref| (test_kernels.py:34-36)


def up(dev, arr, kind="cached"):
    b = dev.buffer(arr.nbytes, kind)
    b.array(arr.dtype, arr.shape)[...] = arr
    b.flush()
    return b


def down(dev, buf, dtype, shape):
    if buf.kind == "device":
        tmp = dev.buffer(buf.size, "cached")
        dev.copy(buf, tmp, buf.size)
        tmp.invalidate()
        out = tmp.array(dtype, shape).copy()
        tmp.destroy()
        return out
    buf.invalidate()
    return buf.array(dtype, shape).copy()


def relerr(got, ref):
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-6))


@pytest.mark.parametrize("i", range(len(mg.MATMUL_CASES)))
def test_reference_kernel_cases(dev, i):
    """test_kernels.py:47-66 shapes through kernels.Matmul with its own buffer kinds."""
    from vkgrad_b200.kernels import Matmul
    m, n, k, ta, tb = mg.MATMUL_CASES[i]
    a, b = mg.matmul_inputs(m, n, k, ta, tb)
    ba, bb = up(dev, a, "shared"), up(dev, b, "shared")
    bc = dev.buffer(m * n * 4, "cached")
    bc.array(np.float32)[:] = np.nan
    bc.flush()
    mm = Matmul(dev, 2, 2, 2, ta, tb)
    mm(ba, bb, bc, m, n, k)
    got = down(dev, bc, np.float32, (m, n))
    z = np.load(os.path.join(GOLD, "matmul.npz"))
    assert relerr(got[::7, ::5], z[f"c{i}_sample"]) < TOL
    assert relerr(got, orc.matmul16(a, b, ta, tb)) < TOL
    for x in (ba, bb, bc):
        x.destroy()


def test_accumulate_is_f32(dev):
    """All-ones 64x64x1024 must be exactly 1024 (test_kernels.py:69-100)."""
    from vkgrad_b200.kernels import Matmul
    m = n = 64
    k = 1024
    ba = up(dev, np.ones((m, k), np.float16), "shared")
    bb = up(dev, np.ones((k, n), np.float16), "shared")
    bc = dev.buffer(m * n * 4, "cached")
    Matmul(dev, 1, 2, 2)(ba, bb, bc, m, n, k)
    got = down(dev, bc, np.float32, (m, n))
    assert np.all(got == float(k))
    for x in (ba, bb, bc):
        x.destroy()


@pytest.mark.parametrize("m,n,k,ta,tb", [
    (32, 16, 32, False, False), (32, 96, 16, False, True), (16, 32, 32, True, False),
    (200, 72, 40, False, False), (136, 264, 200, True, True), (1, 8, 8, False, False),
    (300, 520, 72, False, True), (520, 24, 136, True, False)])
@pytest.mark.parametrize("tile_n", [0, 64, 256])
def test_ragged_shapes(dev, m, n, k, ta, tb, tile_n):
    """Edges that are not tile multiples (the reference raises VkError for these)."""
    from vkgrad_b200.kernels import gemm
    rng = np.random.default_rng(m * 7 + n)
    a = rng.standard_normal((k, m) if ta else (m, k)).astype(np.float16)
    b = rng.standard_normal((n, k) if tb else (k, n)).astype(np.float16)
    ba, bb = up(dev, a), up(dev, b)
    guard = 64
    bc = up(dev, np.full(m * n + guard, np.nan, np.float32))
    gemm(dev, ba, bb, bc, m, n, k, ta, tb, tile_n=tile_n)
    full = down(dev, bc, np.float32, (m * n + guard,))
    assert np.isnan(full[m * n:]).all(), "wrote past the end of C"
    assert relerr(full[:m * n].reshape(m, n), orc.matmul16(a, b, ta, tb)) < TOL
    for x in (ba, bb, bc):
        x.destroy()


def test_misaligned_shape_is_rejected(dev):
    from vkgrad_b200.kernels import Matmul
    from vkgrad_b200.vk import VkError
    ba, bb, bc = (dev.buffer(4096, "device") for _ in range(3))
    with pytest.raises(VkError):
        Matmul(dev)(ba, bb, bc, 16, 12, 16)     # n not a multiple of 8
    with pytest.raises(VkError):
        Matmul(dev)(ba, bb, bc, 16, 16, 20)     # row pitch of A not 16-byte aligned
    for x in (ba, bb, bc):
        x.destroy()


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False)])
def test_batched_dense_stack(dev, ta, tb):
    """kernels.Matmul(batched=True) with element strides (kernels.py:58-64)."""
    from vkgrad_b200.kernels import Matmul
    nb, m, n, k = 6, 64, 48, 32
    rng = np.random.default_rng(5)
    a = rng.standard_normal((nb,) + ((k, m) if ta else (m, k))).astype(np.float16)
    b = rng.standard_normal((nb,) + ((n, k) if tb else (k, n))).astype(np.float16)
    ba, bb = up(dev, a), up(dev, b)
    bc = dev.buffer(nb * m * n * 4, "cached")
    Matmul(dev, 1, 1, 1, ta, tb, batched=True)(ba, bb, bc, m, n, k, nbatch=nb,
                                               strides=(m * k, k * n, m * n))
    got = down(dev, bc, np.float32, (nb, m, n))
    ref = np.stack([orc.matmul16(a[i], b[i], ta, tb) for i in range(nb)])
    assert relerr(got, ref) < TOL
    for x in (ba, bb, bc):
        x.destroy()


def test_heads_addressed_in_place(dev):
    """Q K^T per (batch, head) read straight out of a (rows, 3D) projection, and
    P V written into the merged (rows, D) layout: what Attention does instead of
    split_qkv / merge_heads (tkernels.py:195-300)."""
    from vkgrad_b200._lib import F16
    from vkgrad_b200.kernels import gemm
    B, T, H, hd = 2, 48, 3, 16
    D = H * hd
    rng = np.random.default_rng(9)
    qkv = rng.standard_normal((B * T, 3 * D)).astype(np.float16)
    bq = up(dev, qkv)
    bs = dev.buffer(B * H * T * T * 4, "cached")
    gemm(dev, bq, bq, bs, T, T, hd, trans_b=True, nb0=H, nb1=B, lda=3 * D, ldb=3 * D, ldc=T,
         sa=(hd, T * 3 * D), sb=(hd, T * 3 * D), sc=(T * T, H * T * T), a_off=0, b_off=D)
    got = down(dev, bs, np.float32, (B, H, T, T))
    q = qkv[:, :D].reshape(B, T, H, hd).transpose(0, 2, 1, 3).astype(np.float32)
    k = qkv[:, D:2 * D].reshape(B, T, H, hd).transpose(0, 2, 1, 3).astype(np.float32)
    v = qkv[:, 2 * D:].reshape(B, T, H, hd).transpose(0, 2, 1, 3).astype(np.float32)
    assert relerr(got, q @ k.transpose(0, 1, 3, 2)) < TOL
    p = rng.random((B, H, T, T)).astype(np.float16)
    bp = up(dev, p)
    bo = up(dev, np.zeros((B * T, D), np.float16))
    gemm(dev, bp, bq, bo, T, hd, T, nb0=H, nb1=B, lda=T, ldb=3 * D, ldc=D,
         sa=(T * T, H * T * T), sb=(hd, T * 3 * D), sc=(hd, T * D), b_off=2 * D, c_dtype=F16)
    got = down(dev, bo, np.float16, (B * T, D)).astype(np.float32)
    ref = (p.astype(np.float32) @ v).transpose(0, 2, 1, 3).reshape(B * T, D)
    assert relerr(got, ref) < 2e-3
    for x in (bq, bs, bp, bo):
        x.destroy()


@pytest.mark.parametrize("act", ["gelu", "relu"])
def test_fused_epilogue(dev, act):
    """bias + saved pre-activation + activation + fp16 narrowing in one GEMM; and the
    backward form: activation derivative and residual in the epilogue."""
    from vkgrad_b200._lib import ACT_GELU, ACT_RELU, F16, F32
    from vkgrad_b200.kernels import gemm
    code = {"gelu": ACT_GELU, "relu": ACT_RELU}[act]
    f, df = orc.ACTS[act]
    m, n, k = 200, 136, 72
    rng = np.random.default_rng(2)
    a = rng.standard_normal((m, k)).astype(np.float16)
    w = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float16)
    bias = rng.standard_normal(n).astype(np.float32)
    res = rng.standard_normal((m, n)).astype(np.float32)
    ba, bw, bb, br = up(dev, a), up(dev, w), up(dev, bias), up(dev, res)
    by = dev.buffer(m * n * 2, "cached")
    bz = dev.buffer(m * n * 4, "cached")
    gemm(dev, ba, bw, by, m, n, k, c_dtype=F16, bias=bb, pre=bz, act=code)
    z_ref = orc.matmul16(a, w) + bias
    assert relerr(down(dev, bz, np.float32, (m, n)), z_ref) < 1e-5
    y = down(dev, by, np.float16, (m, n)).astype(np.float32)
    assert relerr(y, f(z_ref)) < 1e-3
    # backward-style epilogue: out = acc * act'(z) + residual, fp32 plus an fp16 copy
    bo = dev.buffer(m * n * 4, "cached")
    bo16 = dev.buffer(m * n * 2, "cached")
    gemm(dev, ba, bw, bo, m, n, k, c_dtype=F32, dact_z=bz, dact=code, residual=br, c2=bo16)
    ref = orc.matmul16(a, w) * df(z_ref) + res
    got = down(dev, bo, np.float32, (m, n))
    if act == "relu":   # derivative flips at z == 0 only; exclude values within rounding of 0
        mask = np.abs(z_ref) > 1e-4
        assert relerr(got[mask], ref[mask]) < 1e-5
    else:
        assert relerr(got, ref) < 1e-5
        assert relerr(down(dev, bo16, np.float16, (m, n)).astype(np.float32), ref) < 1e-3
    for x in (ba, bw, bb, br, by, bz, bo, bo16):
        x.destroy()


def test_bf16_inputs(dev):
    """bf16 operands (the reference has f16 only): checked against bf16-rounded numpy."""
    from vkgrad_b200._lib import BF16
    from vkgrad_b200.kernels import gemm
    m, n, k = 128, 128, 256
    rng = np.random.default_rng(4)

    def to_bf16(x):
        u = x.astype(np.float32).view(np.uint32)
        u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
        return u.astype(np.uint16)

    a32 = rng.standard_normal((m, k)).astype(np.float32)
    b32 = rng.standard_normal((k, n)).astype(np.float32)
    a16, b16 = to_bf16(a32), to_bf16(b32)
    widen = lambda u: (u.astype(np.uint32) << 16).view(np.float32)
    ba, bb = up(dev, a16), up(dev, b16)
    bc = dev.buffer(m * n * 4, "cached")
    gemm(dev, ba, bb, bc, m, n, k, in_dtype=BF16)
    assert relerr(down(dev, bc, np.float32, (m, n)), widen(a16) @ widen(b16)) < TOL
    for x in (ba, bb, bc):
        x.destroy()


def test_large_shape_linearity(dev):
    """At a BASELINE size (4096 x 3072 x 768) the oracle is still quick, and
    linearity gives a size-independent check: (2A) B == 2 (A B) exactly."""
    from vkgrad_b200.kernels import gemm
    m, k, n = 4096, 768, 3072
    rng = np.random.default_rng(1)
    a = rng.standard_normal((m, k)).astype(np.float16)
    w = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float16)
    ba, ba2, bw = up(dev, a), up(dev, (a * np.float16(2)).astype(np.float16)), up(dev, w)
    bc, bc2 = dev.buffer(m * n * 4, "cached"), dev.buffer(m * n * 4, "cached")
    gemm(dev, ba, bw, bc, m, n, k)
    gemm(dev, ba2, bw, bc2, m, n, k)
    c, c2 = down(dev, bc, np.float32, (m, n)), down(dev, bc2, np.float32, (m, n))
    assert np.array_equal(c2, 2 * c)
    assert relerr(c, orc.matmul16(a, w)) < TOL
    for x in (ba, ba2, bw, bc, bc2):
        x.destroy()


@pytest.mark.parametrize("split_k", [0, 1, 2, 5, 16])
@pytest.mark.parametrize("m,n,k,ta,tb", [(256, 264, 4096, True, False), (136, 72, 1000, False, False),
                                         (768, 768, 8192, True, False)])
def test_split_k(dev, m, n, k, ta, tb, split_k):
    """K cut into slices added in a fixed order: same answer as the unsplit GEMM to fp32
    rounding, bit-identical from run to run."""
    from vkgrad_b200.kernels import gemm
    rng = np.random.default_rng(m + k)
    a = rng.standard_normal((k, m) if ta else (m, k)).astype(np.float16)
    b = rng.standard_normal((n, k) if tb else (k, n)).astype(np.float16)
    ba, bb = up(dev, a), up(dev, b)
    ref = orc.matmul16(a, b, ta, tb)
    outs = []
    for _ in range(2):
        bc = up(dev, np.full((m, n), np.nan, np.float32))
        gemm(dev, ba, bb, bc, m, n, k, ta, tb, split_k=split_k)
        outs.append(down(dev, bc, np.float32, (m, n)))
        bc.destroy()
    assert np.array_equal(outs[0], outs[1])
    # fp32 accumulation order differs from numpy's; over K = 8192 that is ~1e-5 of max|C|
    assert relerr(outs[0], ref) < 5e-5
    for x in (ba, bb):
        x.destroy()


@pytest.mark.parametrize("m,n,k,ta,tb", [
    (512, 768, 320, False, True),        # dX = dY W^T: B stored N x K, 96 rows of it per CTA
    (512, 768, 256, False, False),       # Y = X W: B stored K x N, one and a half 64-column groups per CTA
    (768, 384, 1024, True, False),       # dW = X^T dY
    (1000, 520, 200, False, True),       # ragged M, N, K: the last tile has 136 of 192 columns
    (1000, 520, 200, False, False),
    (4096, 768, 3072, False, True),      # more tiles than CTA pairs, long K
])
def test_cta_pair_tiles_192_wide(dev, m, n, k, ta, tb):
    """256 x 192 tiles on CTA pairs (cta_pair = 1, tile_n = 192) against the oracle and, bit for
    bit, against the single-CTA kernel."""
    from vkgrad_b200.kernels import gemm
    rng = np.random.default_rng(m * 5 + n)
    a = rng.standard_normal((k, m) if ta else (m, k)).astype(np.float16)
    b = rng.standard_normal((n, k) if tb else (k, n)).astype(np.float16)
    ba, bb = up(dev, a), up(dev, b)
    outs = []
    for pair, tn in ((-1, 0), (1, 192)):
        bc = dev.buffer(m * n * 4, "cached")
        bc.array(np.float32)[:] = np.nan
        bc.flush()
        gemm(dev, ba, bb, bc, m, n, k, trans_a=ta, trans_b=tb, split_k=1, cta_pair=pair, tile_n=tn)
        outs.append(down(dev, bc, np.float32, (m, n)))
        bc.destroy()
    ref = orc.matmul16(a, b, ta, tb)
    assert relerr(outs[1], ref) < TOL
    assert np.array_equal(outs[0], outs[1])
    for x in (ba, bb):
        x.destroy()


@pytest.mark.parametrize("m,n,k,ta,tb,split_k", [
    (512, 512, 256, False, False, 1),      # Y = X W, B stored K x N
    (512, 768, 320, False, True, 1),       # dX = dY W^T, B stored N x K
    (768, 512, 1024, True, False, 1),      # dW = X^T dY, A stored K x M
    (1000, 520, 200, False, False, 1),     # ragged M, N, K
    (136, 264, 72, False, True, 1),        # a second row block of 8 rows, one tile column and a bit
    (768, 768, 4096, True, False, 4),      # dW with K split over four slices
    (4096, 3072, 768, False, False, 1),    # more tiles than CTA pairs
])
def test_cta_pair_tiles(dev, m, n, k, ta, tb, split_k):
    """256 x 256 tiles on 2-CTA clusters (tcgen05.mma.cta_group::2) against the oracle and,
    bit for bit, against the single-CTA kernel: both accumulate K in the same order."""
    from vkgrad_b200.kernels import gemm
    rng = np.random.default_rng(m * 7 + n)
    a = rng.standard_normal((k, m) if ta else (m, k)).astype(np.float16)
    b = rng.standard_normal((n, k) if tb else (k, n)).astype(np.float16)
    ba, bb = up(dev, a), up(dev, b)
    outs = []
    for pair in (-1, 1):
        bc = dev.buffer(m * n * 4, "cached")
        bc.array(np.float32)[:] = np.nan
        bc.flush()
        gemm(dev, ba, bb, bc, m, n, k, trans_a=ta, trans_b=tb, split_k=split_k, cta_pair=pair)
        outs.append(down(dev, bc, np.float32, (m, n)))
        bc.destroy()
    ref = orc.matmul16(a, b, ta, tb)
    assert relerr(outs[1], ref) < TOL
    if split_k == 1:
        assert np.array_equal(outs[0], outs[1])
    for x in (ba, bb):
        x.destroy()


def test_cta_pair_fused_epilogues(dev):
    """The training step's epilogues on CTA-pair tiles: bias + keep z + GELU + fp16, and
    GELU'(z) scaling with fp16 output, against the single-CTA kernel."""
    from vkgrad_b200._lib import ACT_GELU, F16
    from vkgrad_b200.kernels import gemm
    m, n, k = 640, 512, 192
    rng = np.random.default_rng(3)
    x = rng.standard_normal((m, k)).astype(np.float16)
    w = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float16)
    bias = rng.standard_normal(n).astype(np.float32)
    z_in = rng.standard_normal((m, n)).astype(np.float32)
    bx, bw, bb, bz = up(dev, x), up(dev, w), up(dev, bias), up(dev, z_in)
    res = []
    for pair in (-1, 1):
        y16 = dev.buffer(m * n * 2, "cached")
        z32 = dev.buffer(m * n * 4, "cached")
        d16 = dev.buffer(m * n * 2, "cached")
        gemm(dev, bx, bw, y16, m, n, k, c_dtype=F16, bias=bb, act=ACT_GELU, pre=z32, cta_pair=pair)
        gemm(dev, bx, bw, d16, m, n, k, c_dtype=F16, dact_z=bz, dact=ACT_GELU, cta_pair=pair)
        res.append((down(dev, y16, np.float16, (m, n)), down(dev, z32, np.float32, (m, n)),
                    down(dev, d16, np.float16, (m, n))))
        for b in (y16, z32, d16):
            b.destroy()
    for got, want in zip(res[1], res[0]):
        assert np.array_equal(got, want)
    zref = orc.matmul16(x, w) + bias
    assert relerr(res[1][1], zref) < TOL
    assert relerr(res[1][0].astype(np.float32), orc.gelu(zref)) < 5e-3
    for b in (bx, bw, bb, bz):
        b.destroy()


def test_cta_pair_192_wide_tiles_with_the_steps_epilogues(dev):
    """256 x 192 CTA-pair tiles with the epilogues the training step runs on them: bias +
    residual into the fp32 stream (fc2 forward, B stored K x N) and a plain fp32 dX through the
    transposed weight (B stored N x K), plus an fp16 output, bit for bit against the
    single-CTA kernel; and the library's own choice (cta_pair = 0, tile_n = 0) on a shape wide
    and long enough for it to pick them."""
    from vkgrad_b200._lib import F16
    from vkgrad_b200.kernels import gemm
    m, n, k = 1000, 768, 1600
    rng = np.random.default_rng(17)
    x = rng.standard_normal((m, k)).astype(np.float16)
    w = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float16)
    wt = np.ascontiguousarray(w.T)
    bias = rng.standard_normal(n).astype(np.float32)
    resid = rng.standard_normal((m, n)).astype(np.float32)
    bx, bw, bwt, bb, br = up(dev, x), up(dev, w), up(dev, wt), up(dev, bias), up(dev, resid)
    res = []
    for pair, tn in ((-1, 0), (1, 192)):
        y32 = dev.buffer(m * n * 4, "cached")
        d32 = dev.buffer(m * n * 4, "cached")
        y16 = dev.buffer(m * n * 2, "cached")
        gemm(dev, bx, bw, y32, m, n, k, bias=bb, residual=br, cta_pair=pair, tile_n=tn)
        gemm(dev, bx, bwt, d32, m, n, k, trans_b=True, cta_pair=pair, tile_n=tn)
        gemm(dev, bx, bw, y16, m, n, k, c_dtype=F16, bias=bb, cta_pair=pair, tile_n=tn)
        res.append((down(dev, y32, np.float32, (m, n)), down(dev, d32, np.float32, (m, n)),
                    down(dev, y16, np.float16, (m, n))))
        for b in (y32, d32, y16):
            b.destroy()
    for got, want in zip(res[1], res[0]):
        assert np.array_equal(got, want)
    ref = orc.matmul16(x, w)
    assert relerr(res[1][0], ref + bias + resid) < TOL
    assert relerr(res[1][1], ref) < TOL
    # the library's own choice: 74 pair tiles of 256 x 192 need 4736 rows at N = 768
    m2 = 4864
    x2 = rng.standard_normal((m2, k)).astype(np.float16)
    bx2 = up(dev, x2)
    outs = []
    for pair in (0, -1):
        c = dev.buffer(m2 * n * 4, "cached")
        gemm(dev, bx2, bwt, c, m2, n, k, trans_b=True, cta_pair=pair)
        outs.append(down(dev, c, np.float32, (m2, n)))
        c.destroy()
    assert np.array_equal(outs[0], outs[1])
    assert relerr(outs[0], orc.matmul16(x2, w)) < TOL
    for b in (bx, bw, bwt, bb, br, bx2):
        b.destroy()


def test_cta_pair_batched_bf16(dev):
    """CTA-pair tiles over a batch of matrices with bf16 operands: the batch index walks the
    tensor maps exactly as in the single-CTA kernel."""
    from vkgrad_b200._lib import BF16
    from vkgrad_b200.kernels import gemm
    nb, m, n, k = 3, 384, 320, 136
    rng = np.random.default_rng(11)

    def to_bf16_bits(x):
        u = x.astype(np.float32).view(np.uint32)
        return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)

    a32 = rng.standard_normal((nb, m, k)).astype(np.float32)
    b32 = rng.standard_normal((nb, k, n)).astype(np.float32)
    a16, b16 = to_bf16_bits(a32), to_bf16_bits(b32)
    ar = (a16.astype(np.uint32) << 16).view(np.float32)
    br = (b16.astype(np.uint32) << 16).view(np.float32)
    ba, bb = up(dev, a16), up(dev, b16)
    outs = []
    for pair in (-1, 1):
        bc = dev.buffer(nb * m * n * 4, "cached")
        gemm(dev, ba, bb, bc, m, n, k, nb0=nb, sa=(m * k, 0), sb=(k * n, 0), sc=(m * n, 0),
             in_dtype=BF16, cta_pair=pair)
        outs.append(down(dev, bc, np.float32, (nb, m, n)))
        bc.destroy()
    assert np.array_equal(outs[0], outs[1])
    assert relerr(outs[1], np.einsum("bmk,bkn->bmn", ar, br)) < TOL
    for x in (ba, bb):
        x.destroy()


@pytest.mark.parametrize("m,n,k,pair", [(640, 520, 192, -1), (1000, 264, 72, -1), (640, 520, 192, 1),
                                        (384, 512, 128, 1)])
def test_epilogue_column_sums(dev, m, n, k, pair):
    """colsum: the bias gradient of the layer below comes out of the GEMM that writes its dY
    (fp16, scaled by GELU'(z)); it must equal the column sums of that stored fp16 matrix
    (what transformer.py:30-36 computes in a separate pass), twice in a row bit for bit."""
    from vkgrad_b200._lib import ACT_GELU, F16
    from vkgrad_b200.kernels import gemm
    rng = np.random.default_rng(m + n)
    dy = rng.standard_normal((m, k)).astype(np.float16)
    w = (rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float16)
    z = rng.standard_normal((m, n)).astype(np.float32)
    bdy, bw, bz = up(dev, dy), up(dev, w), up(dev, z)
    sums = []
    for _ in range(2):
        d16 = dev.buffer(m * n * 2, "cached")
        cs = dev.buffer(n * 4, "cached")
        cs.array(np.float32)[:] = np.nan
        cs.flush()
        gemm(dev, bdy, bw, d16, m, n, k, trans_b=True, c_dtype=F16, dact_z=bz, dact=ACT_GELU,
             colsum=cs, cta_pair=pair)
        got = down(dev, d16, np.float16, (m, n)).astype(np.float64)
        sums.append(down(dev, cs, np.float32, (n,)))
        d16.destroy()
        cs.destroy()
    assert np.array_equal(sums[0], sums[1])
    want = got.sum(0)
    assert np.abs(sums[1] - want).max() <= 1e-4 * max(np.abs(want).max(), 1.0)
    assert relerr(got.astype(np.float32), orc.matmul16(dy, w, False, True) * orc.dgelu(z)) < 5e-3
    for b in (bdy, bw, bz):
        b.destroy()


def test_bounded_wait_reports_and_leaves_the_device_usable(dev):
    """Every device-side wait is bounded.  A wait on a barrier nothing arrives on gives up after
    its budget, the kernel returns, the next sync raises VkError, and the device still computes
    a correct GEMM afterwards (no fault, no hang, no lost context)."""
    from vkgrad_b200.kernels import gemm
    from vkgrad_b200.vk import VkError, _check
    _check(dev.lib.vkg_selftest_wait_timeout(dev.handle, 2_000_000), "selftest")   # about 1 ms
    with pytest.raises(VkError, match="wait gave up"):
        dev.sync()
    dev.sync()   # the error word was cleared when it was reported
    m, n, k = 256, 128, 192
    rng = np.random.default_rng(5)
    a = rng.standard_normal((m, k)).astype(np.float16)
    b = rng.standard_normal((k, n)).astype(np.float16)
    ba, bb = up(dev, a), up(dev, b)
    bc = dev.buffer(m * n * 4, "cached")
    gemm(dev, ba, bb, bc, m, n, k)
    assert relerr(down(dev, bc, np.float32, (m, n)), orc.matmul16(a, b)) < TOL
    for x in (ba, bb, bc):
        x.destroy()


@pytest.mark.parametrize("pair", [-1, 1])
def test_grouped_dw_launch_equals_separate_launches(dev, pair):
    """vkg_gemm_group: the dW = X^T dY of several Linears in one launch must give, bit for bit,
    what one unsplit vkg_gemm per Linear gives, and match the oracle."""
    from vkgrad_b200.kernels import gemm, gemm_group
    rows = 1024
    shapes = [(768, 2304), (768, 768), (768, 3072), (3072, 768), (200, 264)]   # (in, out)
    if pair < 0:
        shapes.append((72, 136))       # a single row block: only without CTA pairs
    rng = np.random.default_rng(9)
    xs = [rng.standard_normal((rows, i)).astype(np.float16) for i, _ in shapes]
    dys = [rng.standard_normal((rows, o)).astype(np.float16) for _, o in shapes]
    bx = [up(dev, x) for x in xs]
    bdy = [up(dev, d) for d in dys]
    res = []
    for grouped in (False, True):
        outs = [dev.buffer(i * o * 4, "cached") for i, o in shapes]
        for b in outs:
            b.array(np.uint8)[:] = 0xFF
            b.flush()
        probs = [(bx[j], bdy[j], outs[j], i, o, rows, dict(trans_a=True))
                 for j, (i, o) in enumerate(shapes)]
        if grouped:
            gemm_group(dev, probs, cta_pair=pair)
        else:
            for pr in probs:
                gemm(dev, *pr[:6], split_k=1, cta_pair=-1, **pr[6])
        res.append([down(dev, outs[j], np.float32, shapes[j]) for j in range(len(shapes))])
        for b in outs:
            b.destroy()
    for j in range(len(shapes)):
        assert np.array_equal(res[0][j], res[1][j]), shapes[j]
        assert relerr(res[1][j], orc.matmul16(xs[j], dys[j], True, False)) < TOL
    for b in bx + bdy:
        b.destroy()
