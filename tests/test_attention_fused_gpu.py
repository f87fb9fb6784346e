"""Fused tcgen05 attention (head dimension 64) against numpy: forward output and
log-sum-exp, then the backward kernels' dQ/dK/dV, with the fp16 rounding points of the
unfused path (P and dS rounded before their products)."""

import numpy as np
import pytest

from oracle import vkgrad_numpy as orc

pytestmark = pytest.mark.gpu


def relerr(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-8))


def up(dev, arr):
    b = dev.buffer(arr.nbytes, "cached")
    b.array(arr.dtype, arr.shape)[...] = arr
    b.flush()
    return b


def get(b, dtype, shape):
    b.invalidate()
    return b.array(dtype, shape).copy()


def reference_attention(qkv, B, T, H, scale, seg=None):
    hd = 64
    D = H * hd
    q, k, v = (qkv[:, i * D:(i + 1) * D].astype(np.float32).reshape(B, T, H, hd).transpose(0, 2, 1, 3)
               for i in range(3))
    s = (q @ k.transpose(0, 1, 3, 2)) * scale
    mask = np.tril(np.ones((T, T), bool))[None, None]
    if seg is not None:
        mask = mask & (np.arange(T)[None, None, None, :] >= seg.reshape(B, 1, T, 1))
    s = np.where(mask, s, -np.inf)
    mx = s.max(-1, keepdims=True)
    e = np.exp(s - mx)
    l = e.sum(-1, keepdims=True)
    p = orc.r16(e / l)
    o = (p @ v).transpose(0, 2, 1, 3).reshape(B * T, D)
    lse2 = (mx[..., 0] + np.log(l[..., 0])) / np.log(2.0)
    return q, k, v, p, o, lse2, mask


@pytest.fixture
def one_pass(dev):
    """Switches the forward to the one-pass kernel for the test and back afterwards."""
    from vkgrad_b200._lib import TUNE_ATTN_ONE_PASS
    from vkgrad_b200.vk import _check

    def set_(on):
        _check(dev.lib.vkg_set_tuning(dev.handle, TUNE_ATTN_ONE_PASS, int(on)), "tune")
    yield set_
    set_(0)


@pytest.mark.parametrize("B,T,H", [(1, 128, 1), (2, 320, 2), (1, 1024, 3), (3, 72, 1)])
@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("kernel", ["two_pass", "one_pass", "one_pass_rescaled"])
def test_forward(dev, one_pass, B, T, H, packed, kernel):
    from vkgrad_b200.vk import _check
    one_pass(kernel != "two_pass")
    hd, D = 64, H * 64
    rng = np.random.default_rng(T + H)
    qkv = rng.standard_normal((B * T, 3 * D)).astype(np.float16)
    if kernel == "one_pass_rescaled":
        # scores that grow along the keys by far more than 2^8 from tile to tile: the running
        # reference maximum must move, and O~ and the row sums must be rescaled, several times
        q = np.abs(qkv[:, :D].astype(np.float32)) * 0.5 + 0.5
        ramp = (np.arange(B * T) % T)[:, None] / 8.0
        k = np.abs(qkv[:, D:2 * D].astype(np.float32)) * 0.05 * (1.0 + ramp)
        qkv[:, :D] = q.astype(np.float16)
        qkv[:, D:2 * D] = k.astype(np.float16)
    seg = None
    if packed:
        seg = np.zeros((B, T), np.uint32)
        seg[:, T // 3:] = T // 3
        seg[0, (2 * T) // 3:] = (2 * T) // 3
        seg = seg.reshape(-1)
    scale = 1.0 / np.sqrt(hd)
    bq = up(dev, qkv)
    bo = up(dev, np.full((B * T, D), np.nan, np.float16))
    bl = up(dev, np.full((B * H, T), np.nan, np.float32))
    bs = None if seg is None else up(dev, seg)
    _check(dev.lib.vkg_attn_fwd(dev.handle, bq.dptr, None if bs is None else bs.dptr, bo.dptr,
                                bl.dptr, B, T, H, hd, scale), "attn_fwd")
    dev.sync()
    _, _, _, _, o, lse2, _ = reference_attention(qkv, B, T, H, scale, seg)
    got = get(bo, np.float16, (B * T, D)).astype(np.float32)
    assert np.isfinite(got).all()
    assert relerr(got, o) < 2e-3
    assert np.abs(get(bl, np.float32, (B, H, T)) - lse2).max() < 1e-3
    for x in (bq, bo, bl) + (() if bs is None else (bs,)):
        x.destroy()


# The backward kernels are persistent (one CTA per SM takes several (tile, head, sequence)
# items); the last two cases have 200 and 396 items, i.e. two and three rows of the snake-order
# dealing on 148 SMs, one of them with a ragged last tile, so item boundaries are crossed.
@pytest.mark.parametrize("B,T,H", [(1, 128, 1), (2, 320, 2), (1, 1024, 2), (2, 72, 1),
                                   (5, 600, 8), (3, 384, 44)])
@pytest.mark.parametrize("packed", [False, True])
def test_backward(dev, B, T, H, packed):
    from vkgrad_b200.vk import _check
    hd, D = 64, H * 64
    rng = np.random.default_rng(7 * T + H)
    qkv = rng.standard_normal((B * T, 3 * D)).astype(np.float16)
    dout = (0.1 * rng.standard_normal((B * T, D))).astype(np.float16)
    seg = None
    if packed:
        seg = np.zeros((B, T), np.uint32)
        seg[:, T // 2:] = T // 2
        seg = seg.reshape(-1)
    scale = 1.0 / np.sqrt(hd)
    bq, bdo = up(dev, qkv), up(dev, dout)
    bo = up(dev, np.zeros((B * T, D), np.float16))
    bl = up(dev, np.zeros((B * H, T), np.float32))
    bdelta = up(dev, np.zeros((B * H, T), np.float32))
    bdq = up(dev, np.full((B * T, 3 * D), np.nan, np.float16))
    bs = None if seg is None else up(dev, seg)
    segp = None if bs is None else bs.dptr
    _check(dev.lib.vkg_attn_fwd(dev.handle, bq.dptr, segp, bo.dptr, bl.dptr, B, T, H, hd, scale),
           "attn_fwd")
    outs, sums = [], []
    bdb = up(dev, np.full(3 * D, np.nan, np.float32))
    bsc = dev.buffer(4 * dev.lib.vkg_attn_bwd_dbias_scratch_floats(B, T, H, hd), "device")
    for _ in range(2):
        _check(dev.lib.vkg_attn_bwd(dev.handle, bq.dptr, bdo.dptr, bo.dptr, bl.dptr, segp, bdq.dptr,
                                    bdelta.dptr, bdb.dptr, bsc.dptr, B, T, H, hd, scale), "attn_bwd")
        dev.sync()
        outs.append(get(bdq, np.float16, (B * T, 3 * D)).astype(np.float32))
        sums.append(get(bdb, np.float32, (3 * D,)))
    assert np.array_equal(outs[0], outs[1]), "backward is not deterministic"
    assert np.array_equal(sums[0], sums[1]), "bias gradient is not deterministic"
    got = outs[0]
    # the qkv bias gradient is the column sum of the stored fp16 gradient
    want_db = got.astype(np.float64).sum(0)
    assert np.abs(sums[0] - want_db).max() <= 1e-4 * max(np.abs(want_db).max(), 1.0)
    bdb.destroy()
    bsc.destroy()
    assert np.isfinite(got).all()
    q, k, v, p, o, lse2, mask = reference_attention(qkv, B, T, H, scale, seg)
    dao = dout.astype(np.float32).reshape(B, T, H, hd).transpose(0, 2, 1, 3)
    dv = p.transpose(0, 1, 3, 2) @ dao
    dp = dao @ v.transpose(0, 1, 3, 2)
    ds = orc.r16(p * (dp - (dp * p).sum(-1, keepdims=True)) * scale)
    dq = ds @ k
    dk = ds.transpose(0, 1, 3, 2) @ q
    merge = lambda t: t.transpose(0, 2, 1, 3).reshape(B * T, D)
    for name, ref, sl in (("dq", dq, slice(0, D)), ("dk", dk, slice(D, 2 * D)),
                          ("dv", dv, slice(2 * D, 3 * D))):
        assert relerr(got[:, sl], merge(ref)) < 3e-3, name
    for x in (bq, bdo, bo, bl, bdelta, bdq) + (() if bs is None else (bs,)):
        x.destroy()
