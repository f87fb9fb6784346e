"""Every streaming / row op of the C ABI against numpy, called with the reference's
buffer order and push values through the kernel dictionaries (kernels.make_kernels,
tkernels.make_transformer_kernels)."""

import numpy as np
import pytest

from oracle import vkgrad_numpy as orc

pytestmark = pytest.mark.gpu


def relerr(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-8))


class Pool:
    def __init__(self, dev):
        self.dev, self.bufs = dev, []

    def up(self, arr):
        b = self.dev.buffer(max(arr.nbytes, 16), "cached")
        b.array(arr.dtype, arr.shape)[...] = arr
        b.flush()
        self.bufs.append(b)
        return b

    def out(self, dtype, shape, fill=None):
        n = int(np.prod(shape))
        b = self.dev.buffer(max(n * np.dtype(dtype).itemsize, 16), "cached")
        if fill is not None:
            b.array(dtype, shape)[...] = fill
            b.flush()
        self.bufs.append(b)
        return b

    @staticmethod
    def get(b, dtype, shape):
        b.invalidate()
        return b.array(dtype, shape).copy()

    def close(self):
        for b in self.bufs:
            b.destroy()


@pytest.fixture
def pool(dev):
    p = Pool(dev)
    yield p
    p.close()


@pytest.fixture(scope="module")
def K(dev):
    from vkgrad_b200.kernels import make_kernels
    from vkgrad_b200.tkernels import make_transformer_kernels
    d = dict(make_kernels(dev))
    d.update(make_transformer_kernels(dev))
    return d


def test_bias_gelu_and_backward(dev, pool, K):
    rng = np.random.default_rng(0)
    rows, ncol = 37, 24
    acc = rng.standard_normal((rows, ncol)).astype(np.float32)
    bias = rng.standard_normal(ncol).astype(np.float32)
    z, y = pool.out(np.float32, acc.shape), pool.out(np.float16, acc.shape)
    K["bias_gelu"]([pool.up(acc), pool.up(bias), z, y], acc.size, ncol)
    zr = acc + bias
    assert np.array_equal(pool.get(z, np.float32, acc.shape), zr)
    assert relerr(pool.get(y, np.float16, acc.shape).astype(np.float32), orc.gelu(zr)) < 1e-3
    dy = rng.standard_normal(acc.shape).astype(np.float32)
    dz16, dz32 = pool.out(np.float16, acc.shape), pool.out(np.float32, acc.shape)
    K["bias_gelu_bwd"]([pool.up(dy), z, dz16, dz32], acc.size)
    ref = dy * orc.dgelu(zr)
    assert relerr(pool.get(dz32, np.float32, acc.shape), ref) < 1e-5
    assert relerr(pool.get(dz16, np.float16, acc.shape).astype(np.float32), ref) < 1e-3
    K["bias_gelu_bwd16"]([pool.up(dy), z, dz16], acc.size)
    zo = pool.out(np.float32, acc.shape)
    K["bias"]([pool.up(acc), pool.up(bias), zo], acc.size, ncol)
    assert np.array_equal(pool.get(zo, np.float32, acc.shape), zr)


@pytest.mark.parametrize("nrow,ncol", [(16, 16), (1000, 72), (8192, 768), (33, 50)])
def test_column_sums(dev, pool, K, nrow, ncol):
    rng = np.random.default_rng(1)
    g = rng.standard_normal((nrow, ncol)).astype(np.float32)
    s = pool.out(np.float32, (ncol,))
    K["col_sum"]([pool.up(g), s], ncol, nrow)
    assert relerr(pool.get(s, np.float32, (ncol,)), g.sum(0)) < 1e-5
    # chunked form adds into a zeroed buffer (transformer.py:30-36); twice = deterministic
    g16 = g.astype(np.float16)
    outs = []
    for _ in range(2):
        s2 = pool.out(np.float32, (ncol,), fill=7.0)
        K["col_sum_zero"]([s2], ncol)
        K["col_sum_chunk16"]([pool.up(g16), s2], 32 * ncol, ncol, nrow, 32)
        outs.append(pool.get(s2, np.float32, (ncol,)))
    assert np.array_equal(outs[0], outs[1])
    assert relerr(outs[0], g16.astype(np.float32).sum(0)) < 1e-5
    s3 = pool.out(np.float32, (ncol,), fill=1.0)
    K["col_sum_chunk"]([pool.up(g), s3], 32 * ncol, ncol, nrow, 32)
    assert relerr(pool.get(s3, np.float32, (ncol,)), g.sum(0) + 1.0) < 1e-5


@pytest.mark.parametrize("rows,stride,ncls", [(16, 16, 10), (64, 272, 257), (8, 50272, 50257),
                                              (4, 16384, 16000), (4, 36864, 36001)])
def test_softmax_ce(dev, pool, K, rows, stride, ncls):
    rng = np.random.default_rng(2)
    logits = (3 * rng.standard_normal((rows, stride))).astype(np.float32)
    labels = rng.integers(0, ncls, rows).astype(np.uint32)
    dl16, dl32 = pool.out(np.float16, logits.shape), pool.out(np.float32, logits.shape)
    loss = pool.out(np.float32, (rows,))
    K["softmax_ce"]([pool.up(logits), pool.up(labels), dl16, dl32, loss], rows, stride, ncls)
    lr, g = orc.softmax_ce(logits, labels, ncls)
    assert relerr(pool.get(loss, np.float32, (rows,)), lr) < 1e-5
    got = pool.get(dl32, np.float32, logits.shape)
    assert relerr(got, g) < 1e-4
    assert np.all(got[:, ncls:] == 0)
    w = rng.uniform(0.5, 2, rows).astype(np.float32)
    w[::3] = 0
    K["softmax_ce_w"]([pool.up(logits), pool.up(labels), pool.up(w), dl16, loss], rows, stride, ncls)
    lw, gw = orc.softmax_ce(logits, labels, ncls, weights=w)
    assert relerr(pool.get(loss, np.float32, (rows,)), lw) < 1e-5
    assert relerr(pool.get(dl16, np.float16, logits.shape).astype(np.float32), gw) < 1e-3


@pytest.mark.parametrize("rows,D", [(32, 32), (50, 96), (300, 128), (1000, 768), (64, 1024)])
def test_layernorm_forward_backward(dev, pool, K, rows, D):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((rows, D)).astype(np.float32) * 2 + 0.5
    gam = (1 + 0.2 * rng.standard_normal(D)).astype(np.float32)
    bet = (0.1 * rng.standard_normal(D)).astype(np.float32)
    dy = rng.standard_normal((rows, D)).astype(np.float32)
    bx, bg, bb = pool.up(x), pool.up(gam), pool.up(bet)
    y16, mu, rstd = pool.out(np.float16, x.shape), pool.out(np.float32, (rows,)), pool.out(np.float32, (rows,))
    K["layernorm"]([bx, bg, bb, y16, mu, rstd], rows * 32, D)
    y, xh, r = orc.layernorm_fwd(x, gam, bet)
    assert relerr(pool.get(y16, np.float16, x.shape).astype(np.float32), y) < 1e-3
    assert relerr(pool.get(rstd, np.float32, (rows,)), r) < 1e-5
    # reference-shaped backward: dx, dy*xhat and dy in fp16
    dx, dyxh, dy16 = pool.out(np.float32, x.shape), pool.out(np.float16, x.shape), pool.out(np.float16, x.shape)
    bdy = pool.up(dy)
    K["layernorm_bwd"]([bdy, bx, bg, mu, rstd, dx, dyxh, dy16], rows * 32, D)
    dxr, dgr, dbr = orc.layernorm_bwd(dy, xh, r, gam)
    assert relerr(pool.get(dx, np.float32, x.shape), dxr) < 1e-4
    assert relerr(pool.get(dyxh, np.float16, x.shape).astype(np.float32), dy * xh) < 1e-3
    # fused form: + residual gradient, fp16 copy, dgamma/dbeta in the same pass
    import ctypes as C
    from vkgrad_b200.vk import _check
    lib, h = dev.lib, dev.handle
    dres = rng.standard_normal((rows, D)).astype(np.float32)
    bres = pool.up(dres)
    dx2, dx16 = pool.out(np.float32, x.shape), pool.out(np.float16, x.shape)
    dg, db = pool.out(np.float32, (D,)), pool.out(np.float32, (D,))
    dxs = pool.out(np.float32, (D,))
    with_dxsum = D % 128 == 0 and D <= 1024
    scratch = dev.scratch(lib.vkg_layernorm_bwd_scratch_floats(rows, D) * 4)
    runs = []
    for _ in range(2):
        _check(lib.vkg_layernorm_bwd(h, bdy.dptr, bx.dptr, bg.dptr, mu.dptr, rstd.dptr, bres.dptr,
                                     dx2.dptr, dx16.dptr, None, None, dg.dptr, db.dptr,
                                     dxs.dptr if with_dxsum else None, scratch.dptr, rows, D),
               "ln_bwd")
        dev.sync()
        runs.append((pool.get(dg, np.float32, (D,)), pool.get(db, np.float32, (D,))))
    assert np.array_equal(runs[0][0], runs[1][0]) and np.array_equal(runs[0][1], runs[1][1])
    assert relerr(pool.get(dx2, np.float32, x.shape), dxr + dres) < 1e-4
    assert relerr(pool.get(dx16, np.float16, x.shape).astype(np.float32), dxr + dres) < 1e-3
    assert relerr(runs[0][0], dgr) < 1e-4
    assert relerr(runs[0][1], dbr) < 1e-4
    if with_dxsum:   # column sums of the output: the consuming Dense's bias gradient
        assert relerr(pool.get(dxs, np.float32, (D,)), (dxr + dres).sum(0)) < 1e-4


@pytest.mark.parametrize("T", [16, 64, 200])
def test_attention_softmax(dev, pool, K, T):
    rng = np.random.default_rng(4)
    B, H = 2, 3
    rows = B * H * T
    s = (2 * rng.standard_normal((B, H, T, T))).astype(np.float32)
    scale = 0.37
    p16 = pool.out(np.float16, s.shape)
    bs = pool.up(s)
    K["attn_softmax"]([bs, p16], rows * 32, T, scale)
    mask = np.tril(np.ones((T, T), bool))
    z = np.where(mask, s * scale, -1e30)
    e = np.exp(z - z.max(-1, keepdims=True)) * mask
    p = e / e.sum(-1, keepdims=True)
    got = pool.get(p16, np.float16, s.shape).astype(np.float32)
    assert relerr(got, p) < 1e-3 and np.all(got[..., ~mask] == 0)
    seg = np.zeros((B, T), np.uint32)
    seg[0, T // 3:] = T // 3
    seg[1, T // 2:] = T // 2
    K["attn_softmax_doc"]([bs, pool.up(seg.reshape(-1)), p16], rows * 32, T, H, scale)
    m2 = mask[None, None] & (np.arange(T)[None, None, None, :] >= seg[:, None, :, None])
    z = np.where(m2, s * scale, -1e30)
    e = np.exp(z - z.max(-1, keepdims=True)) * m2
    p2 = e / e.sum(-1, keepdims=True)
    assert relerr(pool.get(p16, np.float16, s.shape).astype(np.float32), p2) < 1e-3
    dp = rng.standard_normal(s.shape).astype(np.float32)
    ph = p.astype(np.float16)
    ds16 = pool.out(np.float16, s.shape)
    K["attn_softmax_bwd"]([pool.up(dp), pool.up(ph), ds16], rows * 32, T, scale)
    pf = ph.astype(np.float32)
    ref = pf * (dp - (dp * pf).sum(-1, keepdims=True)) * scale
    assert relerr(pool.get(ds16, np.float16, s.shape).astype(np.float32), ref) < 1e-3


def test_head_permutes(dev, pool, K):
    rng = np.random.default_rng(5)
    B, T, H, hd = 2, 24, 3, 8
    D, R = H * hd, 2 * 24
    qkv = rng.standard_normal((R, 3 * D)).astype(np.float32)
    bias = rng.standard_normal(3 * D).astype(np.float32)
    q, k, v = (pool.out(np.float16, (B, H, T, hd)) for _ in range(3))
    K["split_qkv"]([pool.up(qkv), pool.up(bias), q, k, v], R * D, D, T, H, hd)
    full = qkv + bias
    for i, b in enumerate((q, k, v)):
        ref = full[:, i * D:(i + 1) * D].reshape(B, T, H, hd).transpose(0, 2, 1, 3)
        assert relerr(pool.get(b, np.float16, (B, H, T, hd)).astype(np.float32), ref) < 1e-3
    hq = rng.standard_normal((B, H, T, hd)).astype(np.float32)
    merged = pool.out(np.float16, (R, D))
    K["merge_heads"]([pool.up(hq), merged], R * D, D, T, H, hd)
    ref = hq.transpose(0, 2, 1, 3).reshape(R, D)
    assert relerr(pool.get(merged, np.float16, (R, D)).astype(np.float32), ref) < 1e-3
    back = pool.out(np.float16, (B, H, T, hd))
    K["split_heads"]([pool.up(ref.astype(np.float32)), back], R * D, D, T, H, hd)
    assert relerr(pool.get(back, np.float16, (B, H, T, hd)).astype(np.float32), hq) < 1e-3
    dqkv = pool.out(np.float16, (R, 3 * D))
    K["merge_qkv_grad"]([pool.up(hq), pool.up(2 * hq), pool.up(3 * hq), dqkv], R * D, D, T, H, hd)
    got = pool.get(dqkv, np.float16, (R, 3 * D)).astype(np.float32)
    assert relerr(got[:, D:2 * D], 2 * ref) < 1e-3 and relerr(got[:, 2 * D:], 3 * ref) < 1e-3


def test_embedding(dev, pool, K):
    rng = np.random.default_rng(6)
    B, T, D, V = 2, 16, 24, 40
    tok = rng.standard_normal((V, D)).astype(np.float32)
    pos = rng.standard_normal((T, D)).astype(np.float32)
    ids = rng.integers(0, V, B * T).astype(np.uint32)
    x = pool.out(np.float32, (B * T, D))
    K["embed"]([pool.up(tok), pool.up(pos), pool.up(ids), x], B * T * D, D, T)
    t = np.arange(B * T) % T
    assert np.array_equal(pool.get(x, np.float32, (B * T, D)), tok[ids] + pos[t])
    dx = rng.standard_normal((B * T, D)).astype(np.float32)
    dtok, dpos = pool.out(np.float32, tok.shape, fill=0), pool.out(np.float32, pos.shape, fill=0)
    K["embed_bwd"]([pool.up(dx), pool.up(ids), dtok, dpos], B * T * D, D, T)
    rt, rp = np.zeros_like(tok), np.zeros_like(pos)
    np.add.at(rt, ids, dx)
    np.add.at(rp, t, dx)
    assert relerr(pool.get(dtok, np.float32, tok.shape), rt) < 1e-5
    assert relerr(pool.get(dpos, np.float32, pos.shape), rp) < 1e-5
    seg = np.zeros(B * T, np.uint32)
    seg[5:T] = 5
    K["embed_doc"]([pool.up(tok), pool.up(pos), pool.up(ids), pool.up(seg), x], B * T * D, D, T)
    assert np.array_equal(pool.get(x, np.float32, (B * T, D)), tok[ids] + pos[t - seg])


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("B,T,D,V", [(2, 16, 128, 7), (3, 130, 256, 40), (8, 1024, 768, 50257)])
def test_embedding_backward_without_atomics(dev, pool, B, T, D, V, packed):
    """vkg_embed_bwd_det: the scatter-add of tkernels.py:317-360 with the rows of one table row
    added in row order -- equal to a sequential sum bit for bit, twice in a row, also with
    many repeated tokens, packed samples and a table that already holds a gradient."""
    from vkgrad_b200.vk import _check
    rng = np.random.default_rng(B * T + D)
    R = B * T
    ids = rng.integers(0, V, R).astype(np.uint32)
    ids[:: 3] = ids[0]                       # a long chain as well as short ones
    seg = np.zeros(R, np.uint32)
    if packed:
        for b in range(B):
            cut = int(rng.integers(1, T))
            seg[b * T + cut:(b + 1) * T] = cut
    dx = rng.standard_normal((R, D)).astype(np.float32)
    tok0 = rng.standard_normal((V, D)).astype(np.float32)     # the tied head's share
    t = np.arange(R) % T - seg.astype(np.int64)
    rt, rp = tok0.copy(), np.zeros((T, D), np.float32)
    # sequential fp32 sums per table row, rows in increasing order, then one add into the table
    acc_t, acc_p = {}, {}
    for r in range(R):
        k = int(ids[r])
        acc_t[k] = dx[r].copy() if k not in acc_t else acc_t[k] + dx[r]
        k = int(t[r])
        acc_p[k] = dx[r].copy() if k not in acc_p else acc_p[k] + dx[r]
    for k, v in acc_t.items():
        rt[k] = rt[k] + v
    for k, v in acc_p.items():
        rp[k] = rp[k] + v
    lib, h = dev.lib, dev.handle
    scratch = dev.buffer(lib.vkg_embed_bwd_scratch_bytes(R), "device")
    pool.bufs.append(scratch)
    dxb, idb = pool.up(dx), pool.up(ids)
    segb = pool.up(seg) if packed else None
    for _ in range(2):
        dtok, dpos = pool.up(tok0), pool.out(np.float32, (T, D), fill=0)
        _check(lib.vkg_embed_bwd_det(h, dxb.dptr, idb.dptr, None if segb is None else segb.dptr,
                                     dtok.dptr, dpos.dptr, scratch.dptr, R * D, D, T), "embed_bwd_det")
        assert np.array_equal(pool.get(dtok, np.float32, (V, D)), rt)
        assert np.array_equal(pool.get(dpos, np.float32, (T, D)), rp)


def test_residual_add_cast(dev, pool, K):
    rng = np.random.default_rng(7)
    R, D = 33, 40
    a, r = (rng.standard_normal((R, D)).astype(np.float32) for _ in range(2))
    bias = rng.standard_normal(D).astype(np.float32)
    o = pool.out(np.float32, (R, D))
    K["residual"]([pool.up(a), pool.up(bias), pool.up(r), o], R * D, D)
    assert np.allclose(pool.get(o, np.float32, (R, D)), r + a + bias, atol=1e-6)
    K["add"]([pool.up(a), pool.up(r), o], R * D)
    assert np.array_equal(pool.get(o, np.float32, (R, D)), a + r)
    xa = pool.up(a)
    K["add_bias"]([xa, pool.up(bias)], R * D, D)
    assert np.array_equal(pool.get(xa, np.float32, (R, D)), a + bias)
    h = pool.out(np.float16, (R, D))
    K["to16"]([pool.up(a), h], R * D)
    assert np.array_equal(pool.get(h, np.float16, (R, D)), a.astype(np.float16))
    K["cast16"]([pool.up(a), h], R * D)
    assert np.array_equal(pool.get(h, np.float16, (R, D)), a.astype(np.float16))
    zbuf = pool.out(np.float32, (R, D), fill=3.0)
    K["zero"]([zbuf], R * D)
    assert not pool.get(zbuf, np.float32, (R, D)).any()


def test_adamw_single_and_multi_tensor(dev, pool, K):
    """K["adamw"] per tensor (kernels.py:832-851) and the one-launch table form give
    the oracle's update; odd sizes exercise the vector tail."""
    import ctypes as C
    from vkgrad_b200.vk import _check
    rng = np.random.default_rng(8)
    sizes = [4096 * 3 + 5, 17, 768, 4099]
    lr, b1, b2, eps, t = 3e-3, 0.9, 0.999, 1e-8, 4
    bc1, bc2 = orc.adamw_bias_corrections(t, b1, b2)
    hp = dev.buffer(32, "shared")
    hp.array(np.float32)[:] = [lr, b1, b2, bc1, bc2, eps, 0.5, 0]
    tensors = []
    for n in sizes:
        w = rng.standard_normal(n).astype(np.float32)
        g = rng.standard_normal(n).astype(np.float32)
        m = (0.1 * rng.standard_normal(n)).astype(np.float32)
        v = np.abs(0.01 * rng.standard_normal(n)).astype(np.float32)
        tensors.append((w, g, m, v))
    for mode in ("single", "multi"):
        bufs = [[pool.up(a) for a in tns] + [pool.out(np.float16, (len(tns[0]),))] for tns in tensors]
        wds = [0.01, 0.0, 0.01, 0.0]
        if mode == "single":
            for (bw, bg, bm, bv, b16), n, wd in zip(bufs, sizes, wds):
                K["adamw"]([bw, bg, bm, bv, b16, hp], n, wd)
        else:
            n = len(sizes)
            arr = lambda i: (C.c_void_p * n)(*[b[i].dptr for b in bufs])
            tab = C.c_void_p()
            _check(dev.lib.vkg_adamw_table_create(dev.handle, n, arr(0), arr(1), arr(2), arr(3), arr(4),
                                                  (C.c_int64 * n)(*sizes), (C.c_float * n)(*wds),
                                                  C.byref(tab)), "table")
            _check(dev.lib.vkg_adamw_multi(dev.handle, tab, hp.dptr), "multi")
            dev.sync()
            _check(dev.lib.vkg_adamw_table_destroy(dev.handle, tab), "destroy")
        for (bw, bg, bm, bv, b16), (w, g, m, v), wd in zip(bufs, tensors, wds):
            wr, mr, vr, w16 = orc.adamw_step(w, g, m, v, t, lr, b1, b2, eps, wd, gscale=0.5)
            n = len(w)
            assert np.abs(pool.get(bw, np.float32, (n,)) - wr).max() < 2e-6, mode
            assert np.abs(pool.get(bm, np.float32, (n,)) - mr).max() < 1e-6
            assert np.abs(pool.get(bv, np.float32, (n,)) - vr).max() < 1e-6
            got16 = pool.get(b16, np.float16, (n,))
            assert np.array_equal(got16, pool.get(bw, np.float32, (n,)).astype(np.float16))
    hp.destroy()


def test_gradient_exchange_kernels(dev, pool):
    """push/add, zero, pull with the reference's (buffers, n, off[, scale]) convention."""
    from vkgrad_b200.dataparallel import make_reduce_kernels
    R = make_reduce_kernels(dev)
    g = np.arange(10, dtype=np.float32)
    arena = pool.out(np.float32, (32,), fill=5.0)
    R["zero"]([arena], 32)
    R["push"]([pool.up(g), arena], 10, 4)
    R["add"]([pool.up(g), arena], 10, 4)
    a = pool.get(arena, np.float32, (32,))
    assert np.array_equal(a[4:14], 2 * g) and not a[:4].any() and not a[14:].any()
    out = pool.out(np.float32, (10,))
    R["pull"]([arena, out], 10, 4, 0.25)
    assert np.array_equal(pool.get(out, np.float32, (10,)), 0.5 * g)


def test_bucket_pack_roundtrip(dev, pool):
    from vkgrad_b200._lib import BF16, F16
    from vkgrad_b200.vk import _check
    x = np.linspace(-4, 4, 1000).astype(np.float32)
    bx = pool.up(x)
    for dt in (F16, BF16):
        b16, back = pool.out(np.float16, (1000,)), pool.out(np.float32, (1000,))
        _check(dev.lib.vkg_bucket_pack16(dev.handle, bx.dptr, b16.dptr, dt, 1000, 8.0), "pack")
        _check(dev.lib.vkg_bucket_unpack16(dev.handle, b16.dptr, dt, back.dptr, 1000, 0.125), "unpack")
        dev.sync()
        assert relerr(pool.get(back, np.float32, (1000,)), x) < (1e-3 if dt == F16 else 8e-3)


def test_deferred_final_passes_equal_immediate_ones(dev, pool, K):
    """vkg_finals_defer / vkg_finals_flush: layernorm-parameter sums and a column sum whose
    second passes are collected and run as one launch give what the immediate passes give
    (to rounding: the collected pass adds each column in 32 slices, the stand-alone column
    sum in 8), nothing is written before the flush, and a pending list refuses to be
    switched off."""
    import ctypes as C
    from vkgrad_b200.vk import VkError, _check
    lib, h = dev.lib, dev.handle
    rows, D = 1024, 256
    rng = np.random.default_rng(11)
    x = rng.standard_normal((rows, D)).astype(np.float32)
    dy = rng.standard_normal((rows, D)).astype(np.float32)
    gamma = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    mu = x.mean(1).astype(np.float32)
    rstd = (1 / np.sqrt(x.var(1) + 1e-5)).astype(np.float32)

    def up(a):
        b = dev.buffer(a.nbytes, "cached")
        b.array(a.dtype, a.shape)[...] = a
        b.flush()
        return b

    def down(b, shape):
        b.invalidate()
        return b.array(np.float32, shape).copy()

    bx, bdy, bg, bmu, brs = up(x), up(dy), up(gamma), up(mu), up(rstd)
    dx, dx16 = dev.buffer(rows * D * 4, "device"), dev.buffer(rows * D * 2, "device")
    n_sc = lib.vkg_layernorm_bwd_scratch_floats(rows, D)
    results = []
    for deferred in (False, True):
        dg, db, dxs = (up(np.full(D, np.nan, np.float32)) for _ in range(3))
        sc1, sc2 = dev.buffer(n_sc * 4, "device"), dev.buffer(n_sc * 4, "device")
        if deferred:
            _check(lib.vkg_finals_defer(h, 1), "defer")
        # two producers with scratch of their own, as deferral demands
        _check(lib.vkg_layernorm_bwd(h, bdy.dptr, bx.dptr, bg.dptr, bmu.dptr, brs.dptr, None, dx.dptr,
                                     dx16.dptr, None, None, dg.dptr, db.dptr, dxs.dptr, sc1.dptr,
                                     rows, D), "ln_bwd")
        dg2, db2 = up(np.full(D, np.nan, np.float32)), up(np.full(D, np.nan, np.float32))
        _check(lib.vkg_layernorm_bwd(h, bx.dptr, bdy.dptr, bg.dptr, bmu.dptr, brs.dptr, None, dx.dptr,
                                     dx16.dptr, None, None, dg2.dptr, db2.dptr, None, sc2.dptr,
                                     rows, D), "ln_bwd 2")
        if deferred:
            dev.sync()
            assert np.isnan(down(dg, (D,))).all(), "written before the flush"
            assert lib.vkg_finals_defer(h, 0) != 0          # two passes are pending
            _check(lib.vkg_finals_flush(h), "flush")
            _check(lib.vkg_finals_flush(h), "empty flush")   # nothing left: no launch, no error
        dev.sync()
        results.append([down(b, (D,)) for b in (dg, db, dxs, dg2, db2)])
        for b in (dg, db, dxs, dg2, db2, sc1, sc2):
            b.destroy()
    for a, b in zip(*results):
        assert np.isfinite(a).all() and np.isfinite(b).all()
        assert np.abs(a - b).max() <= 1e-5 * max(np.abs(a).max(), 1.0)
    # against numpy: dbeta = column sums of dy
    assert np.abs(results[1][1] - dy.sum(0)).max() < 1e-3
    assert np.abs(results[1][4] - x.sum(0)).max() < 1e-3
    # switching off with nothing pending is fine; -1 drops pending passes
    _check(lib.vkg_finals_defer(h, 1), "defer")
    sc = dev.buffer(n_sc * 4, "device")
    dg, db = up(np.zeros(D, np.float32)), up(np.zeros(D, np.float32))
    _check(lib.vkg_layernorm_bwd(h, bdy.dptr, bx.dptr, bg.dptr, bmu.dptr, brs.dptr, None, dx.dptr,
                                 dx16.dptr, None, None, dg.dptr, db.dptr, None, sc.dptr, rows, D), "ln")
    _check(lib.vkg_finals_defer(h, -1), "drop")
    _check(lib.vkg_finals_defer(h, 0), "off")
    dev.sync()
    assert not down(dg, (D,)).any()
    for b in (bx, bdy, bg, bmu, brs, dx, dx16, sc, dg, db):
        b.destroy()

